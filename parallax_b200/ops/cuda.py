"""Torch-tensor wrappers over the sm_100a kernel library.

Every function here launches hand-written CUDA kernels on the current CUDA stream of the
tensors' device. Shapes and semantics are documented with the C ABI in ``csrc/pxl_api.h``.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _lib
from ._lib import EPI_F32, EPI_NONE, EPI_RESIDUAL, EPI_SILU_MUL, check

_status: dict[int, torch.Tensor] = {}
_workspaces: dict[tuple[int, str], torch.Tensor] = {}
launch_count = 0  # number of kernel-library launches issued (benchmarks report it)


_CHECK_EACH_OP = bool(os.environ.get("PXL_CHECK_EACH_OP"))
_PREFILL_LEGACY = bool(os.environ.get("PXL_PREFILL_LEGACY"))    # mma.sync prefill attention instead of tcgen05


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n
    if _CHECK_EACH_OP:
        # debugging aid: synchronise after every op and name the op whose kernel reported an error
        import sys

        for idx, t in _status.items():
            code = int(t.item())
            if code:
                t.zero_()
                raise _lib.KernelError(f"{sys._getframe(1).f_code.co_name} on cuda:{idx}: {_lib.describe(code)}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def status_tensor(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels set instead of trapping (0 = healthy)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        with torch.inference_mode(False):      # a normal tensor: it is reset in place from any context
            t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device: torch.device) -> None:
    """Synchronising read of the device status word; raises if a kernel reported an error."""
    code = int(status_tensor(device).item())
    if code != 0:
        status_tensor(device).zero_()
        raise _lib.KernelError(f"device status: {_lib.describe(code)}")


_status_host: dict[int, torch.Tensor] = {}


def status_copy_async(device: torch.device) -> None:
    """Enqueue a copy of the status word into a pinned host mirror on the current stream. The
    serving loops call this right before the step's device-to-host token copy, so the mirror is
    valid once the tokens are: reading it costs no synchronisation of its own."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    h = _status_host.get(idx)
    if h is None:
        with torch.inference_mode(False):
            h = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        _status_host[idx] = h
    h.copy_(status_tensor(device), non_blocking=True)


def status_mirror(device: torch.device) -> int:
    """Value that the last completed :func:`status_copy_async` brought back (0 = healthy)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    h = _status_host.get(idx)
    return int(h[0]) if h is not None else 0


def raise_if_status(device: torch.device) -> None:
    """Raise (and clear the word) if the mirrored status is non-zero. After a non-zero status the
    output of the kernels of that step is undefined: the caller fails the batch."""
    code = status_mirror(device)
    if code != 0:
        status_tensor(device).zero_()
        _status_host[device.index if device.index is not None else torch.cuda.current_device()].zero_()
        raise _lib.KernelError(f"device status: {_lib.describe(code)}")


def workspace(device: torch.device, tag: str, nbytes: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, tag)
    t = _workspaces.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", idx))
        _workspaces[key] = t
    return t


# ----------------------------------------------------------------------------- GEMM
def linear(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    epi: int = EPI_NONE,
    out: Optional[torch.Tensor] = None,
    bn: int = 0,
) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T`` on tcgen05 tensor cores with a fused epilogue."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1]
    assert x.stride(1) == 1 and w.stride(1) == 1
    M, K = x.shape
    N = w.shape[0]
    if residual is not None:
        epi = EPI_RESIDUAL
    n_out = N // 2 if epi == EPI_SILU_MUL else N
    if out is None:
        out = torch.empty(
            (M, n_out), dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=x.device
        )
    if M == 0:
        return out
    if residual is not None:
        assert residual.shape == out.shape and residual.stride(0) == out.stride(0)
    code = _lib.lib().pxl_gemm_bf16(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual), _ptr(bias), M, N, K,
        x.stride(0), w.stride(0), out.stride(0), epi, bn, status_tensor(x.device).data_ptr(),
        _stream(x.device),
    )
    check(code, "pxl_gemm_bf16")
    _count()
    return out


def gemm_pick_bn(M: int, N: int, epi: int = EPI_NONE) -> int:
    return _lib.lib().pxl_gemm_bf16_pick_bn(M, N, epi)


def gemm_uses_small_m(M: int, N: int, K: int, epi: int = EPI_NONE) -> bool:
    """Whether :func:`linear` (automatic tile choice) runs this shape on the small-M split-K path."""
    return bool(_lib.lib().pxl_gemm_bf16_uses_small_m(M, N, K, epi))


def linear_small_m(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   residual: Optional[torch.Tensor] = None, splitk: int = 0,
                   out: Optional[torch.Tensor] = None, mode: int = 0) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T`` for M <= 128 on the swapped-operand split-K kernel (``splitk`` 0 = automatic;
    ``mode`` 1 = partial sums through a global scratch, 2 = reduced inside a thread-block cluster over
    distributed shared memory, 0 = automatic). :func:`linear` picks this path by itself; the explicit
    entry exists for tests and benchmarks."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] == w.shape[1]
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if residual is not None:
        assert residual.shape == out.shape and residual.stride(0) == out.stride(0)
    code = _lib.lib().pxl_gemm_bf16_small_m(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual), _ptr(bias), M, N, K, x.stride(0), w.stride(0),
        out.stride(0), splitk, mode, status_tensor(x.device).data_ptr(), _stream(x.device))
    check(code, "pxl_gemm_bf16_small_m")
    _count()
    return out


def gemm_mid_m_plan(M: int, N: int, K: int, epi: int = EPI_NONE) -> tuple[int, int]:
    """``(tile width, K ranges)`` that :func:`linear` picks for 128 < M <= 1024 rows; K ranges == 1 means the
    plain persistent kernel, ``(0, 0)`` that the shape is outside the mid-M range."""
    code = _lib.lib().pxl_gemm_bf16_mid_m_plan(M, N, K, epi)
    return (code >> 4, code & 15)


def linear_mid_m(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, bn: int = 256, splitk: int = 2,
                 out: Optional[torch.Tensor] = None, f32: bool = False) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T`` on the mid-M kernel: 128-row token tiles, the K ranges of a tile spread over
    a thread-block cluster and reduced through distributed shared memory. :func:`linear` picks this path
    by itself; the explicit entry exists for tests and benchmarks."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] == w.shape[1]
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
    if residual is not None:
        assert residual.shape == out.shape and residual.stride(0) == out.stride(0)
    code = _lib.lib().pxl_gemm_bf16_mid_m(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual), _ptr(bias), M, N, K, x.stride(0), w.stride(0),
        out.stride(0), bn, splitk, 1 if f32 else 0, status_tensor(x.device).data_ptr(), _stream(x.device))
    check(code, "pxl_gemm_bf16_mid_m")
    _count()
    return out


# ---------------------------------------------------------------------- elementwise
def rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    residual: Optional[torch.Tensor] = None,
    w_offset: float = 0.0,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    T, H = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    if out is None:
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    if not x.is_contiguous() or not out.is_contiguous():
        # rows of a column slice (e.g. the q part of a packed qkv activation); out may alias x
        assert residual is None and out.stride(1) == 1
        check(_lib.lib().pxl_rmsnorm_strided(x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0),
                                             T, H, eps, w_offset, _stream(x.device)), "pxl_rmsnorm_strided")
        _count()
        return out
    check(
        _lib.lib().pxl_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), _ptr(residual), T,
                               H, eps, w_offset, _stream(x.device)),
        "pxl_rmsnorm",
    )
    _count()
    return out


def _is_fp8_cache(t: Optional[torch.Tensor]) -> bool:
    return t is not None and t.dtype == torch.float8_e4m3fn


def qk_norm_rope_cache(
    qkv: torch.Tensor,
    q_norm_w: Optional[torch.Tensor],
    k_norm_w: Optional[torch.Tensor],
    cos_sin: Optional[torch.Tensor],
    positions: torch.Tensor,
    slot_mapping: Optional[torch.Tensor],
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rot_dim: int,
    eps: float = 1e-6,
    norm_w_offset: float = 0.0,
    kv_scale: tuple = (1.0, 1.0),
) -> None:
    """In place on ``qkv``: per-head norm + RoPE for q and k; k, v scattered to the cache (bf16, or e4m3
    bytes divided by ``kv_scale`` when the cache tensors are ``float8_e4m3fn``)."""
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (num_q_heads + 2 * num_kv_heads) * head_dim
    assert positions.dtype == torch.int32
    if slot_mapping is not None:
        assert slot_mapping.dtype == torch.int64
    page = k_cache.shape[2] if k_cache is not None else 1
    slots = k_cache.shape[0] * page if k_cache is not None else 0
    if cos_sin is None:
        rot_dim = 0
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    if _is_fp8_cache(k_cache):
        check(
            _lib.lib().pxl_qk_norm_rope_cache_fp8(
                qkv.data_ptr(), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos_sin), positions.data_ptr(),
                _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), T, num_q_heads, num_kv_heads,
                head_dim, rot_dim, page, slots, eps, norm_w_offset, float(kv_scale[0]), float(kv_scale[1]),
                max_pos, status_tensor(qkv.device).data_ptr(), _stream(qkv.device)),
            "pxl_qk_norm_rope_cache_fp8",
        )
        _count()
        return
    check(
        _lib.lib().pxl_qk_norm_rope_cache(
            qkv.data_ptr(), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos_sin), positions.data_ptr(),
            _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), T, num_q_heads, num_kv_heads,
            head_dim, rot_dim, page, slots, eps, norm_w_offset, max_pos,
            status_tensor(qkv.device).data_ptr(), _stream(qkv.device)),
        "pxl_qk_norm_rope_cache",
    )
    _count()


def reshape_and_cache(
    k: Optional[torch.Tensor],
    v: Optional[torch.Tensor],
    slot_mapping: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    kv_scale: tuple = (1.0, 1.0),
) -> None:
    """Scatter k, v ``[T, H, D]`` into paged caches ``[blocks, H, page, D]`` (bf16 or scaled e4m3)."""
    ref = k if k is not None else v
    T = ref.shape[0]
    cache = k_cache if k_cache is not None else v_cache
    Hkv, page = cache.shape[1], cache.shape[2]
    Dk = k_cache.shape[3] if k_cache is not None else 0
    Dv = v_cache.shape[3] if v_cache is not None else 0
    if _is_fp8_cache(cache):
        check(
            _lib.lib().pxl_reshape_and_cache_fp8(
                _ptr(k), _ptr(v), k.stride(0) if k is not None else 0,
                v.stride(0) if v is not None else 0, slot_mapping.data_ptr(), _ptr(k_cache),
                _ptr(v_cache), T, Hkv, Dk, Dv, page, cache.shape[0] * page, float(kv_scale[0]),
                float(kv_scale[1]), status_tensor(ref.device).data_ptr(), _stream(ref.device)),
            "pxl_reshape_and_cache_fp8",
        )
        _count()
        return
    check(
        _lib.lib().pxl_reshape_and_cache(
            _ptr(k), _ptr(v), k.stride(0) if k is not None else 0,
            v.stride(0) if v is not None else 0, slot_mapping.data_ptr(), _ptr(k_cache),
            _ptr(v_cache), T, Hkv, Dk, Dv, page, cache.shape[0] * page,
            status_tensor(ref.device).data_ptr(), _stream(ref.device)),
        "pxl_reshape_and_cache",
    )
    _count()


def act_mul(x: torch.Tensor, mode: int = 0, limit: float = 7.0) -> torch.Tensor:
    T, I2 = x.shape
    out = torch.empty((T, I2 // 2), dtype=x.dtype, device=x.device)
    check(_lib.lib().pxl_act_mul(x.data_ptr(), out.data_ptr(), T, I2 // 2, mode, limit,
                                 _stream(x.device)), "pxl_act_mul")
    _count()
    return out


def patch_ids(dst: torch.Tensor, dst_idx: torch.Tensor, src: torch.Tensor, src_idx: torch.Tensor) -> None:
    """``dst[dst_idx] = src[src_idx]`` on int32 tensors (token ids that never left the device)."""
    n = dst_idx.numel()
    if n == 0:
        return
    assert dst.dtype == src.dtype == dst_idx.dtype == src_idx.dtype == torch.int32
    check(_lib.lib().pxl_patch_i32(dst.data_ptr(), dst_idx.data_ptr(), src.data_ptr(), src_idx.data_ptr(), n,
                                   dst.numel(), src.numel(), status_tensor(dst.device).data_ptr(), _stream(dst.device)),
          "pxl_patch_i32")
    _count()


def gather_rows(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, H = ids.numel(), table.shape[1]
    assert table.is_contiguous() and ids.dtype in (torch.int32, torch.int64)
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    check(
        _lib.lib().pxl_gather_rows(table.data_ptr(), ids.data_ptr(), out.data_ptr(), T, H,
                                   table.shape[0], int(ids.dtype == torch.int64),
                                   status_tensor(table.device).data_ptr(), _stream(table.device)),
        "pxl_gather_rows",
    )
    _count()
    return out


def add_inplace(y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    assert y.is_contiguous() and x.is_contiguous() and y.numel() == x.numel()
    check(_lib.lib().pxl_add_inplace(y.data_ptr(), x.data_ptr(), y.numel(), _stream(y.device)),
          "pxl_add_inplace")
    _count()
    return y


# ------------------------------------------------------------------------ attention
def attn_decode(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    ctx_lens: torch.Tensor,
    scale: float,
    window: int = 0,
    sinks: Optional[torch.Tensor] = None,
    max_ctx: int = 0,
    num_splits: int = 0,
    out: Optional[torch.Tensor] = None,
    kv_scale: tuple = (1.0, 1.0),
) -> torch.Tensor:
    """q ``[B, Hq, D]`` (may be a strided view into a packed qkv buffer) vs the paged cache (bf16, or e4m3
    with ``kv_scale``)."""
    B, Hq, D = q.shape
    assert q.stride(2) == 1 and q.stride(1) == D
    Hkv, page = k_cache.shape[1], k_cache.shape[2]
    if out is None:
        out = torch.empty((B, Hq, D), dtype=q.dtype, device=q.device)
    if max_ctx <= 0:
        max_ctx = block_tables.shape[1] * page
    if num_splits <= 0:
        num_splits = _lib.lib().pxl_attn_decode_splits(B, Hkv, max_ctx)
    ws = None
    if num_splits > 1:
        ws = workspace(q.device, "attn_decode", B * Hq * num_splits * (D + 2) * 4)
    if _is_fp8_cache(k_cache):
        check(
            _lib.lib().pxl_attn_decode_fp8(
                q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                block_tables.data_ptr(), ctx_lens.data_ptr(), out.data_ptr(), _ptr(ws), _ptr(sinks),
                B, Hq, Hkv, D, page, block_tables.shape[1], k_cache.shape[0], scale, window, num_splits, max_ctx,
                float(kv_scale[0]), float(kv_scale[1]), status_tensor(q.device).data_ptr(), _stream(q.device)),
            "pxl_attn_decode_fp8",
        )
        _count(2 if num_splits > 1 else 1)
        return out
    check(
        _lib.lib().pxl_attn_decode(
            q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            block_tables.data_ptr(), ctx_lens.data_ptr(), out.data_ptr(), _ptr(ws), _ptr(sinks),
            B, Hq, Hkv, D, page,
            block_tables.shape[1], k_cache.shape[0], scale, window, num_splits, max_ctx,
            status_tensor(q.device).data_ptr(), _stream(q.device)),
        "pxl_attn_decode",
    )
    _count(2 if num_splits > 1 else 1)
    return out


def attn_prefill(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    cu_q: torch.Tensor,
    ctx_lens: torch.Tensor,
    max_q_len: int,
    scale: float,
    window: int = 0,
    sinks: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    kv_scale: tuple = (1.0, 1.0),
) -> torch.Tensor:
    """q ``[T, Hq, D]`` (may be a strided view into a packed qkv buffer)."""
    T, Hq, D = q.shape
    assert q.stride(2) == 1 and q.stride(1) == D
    Hkv, page = k_cache.shape[1], k_cache.shape[2]
    if out is None:
        out = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
    B = ctx_lens.numel()
    if T == 0 or B == 0:
        return out
    if _is_fp8_cache(k_cache):
        check(
            _lib.lib().pxl_attn_prefill_fp8(
                q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                block_tables.data_ptr(), cu_q.data_ptr(), ctx_lens.data_ptr(), out.data_ptr(),
                out.stride(0), _ptr(sinks), B, max_q_len, Hq, Hkv, D, page, block_tables.shape[1],
                k_cache.shape[0], scale, window, float(kv_scale[0]), float(kv_scale[1]),
                status_tensor(q.device).data_ptr(), _stream(q.device)),
            "pxl_attn_prefill_fp8",
        )
        _count()
        return out
    if D == 128 and page in (16, 32, 64) and not _PREFILL_LEGACY and q.stride(0) % 8 == 0 \
            and q.data_ptr() % 16 == 0 and out.stride(1) == D and k_cache.shape[0] * Hkv * page < (1 << 31):
        # tcgen05 kernel: query tile, K and V pages through TMA, scores and P V on the tensor cores
        check(
            _lib.lib().pxl_attn_prefill_tc(
                q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                block_tables.data_ptr(), cu_q.data_ptr(), ctx_lens.data_ptr(), out.data_ptr(),
                out.stride(0), _ptr(sinks), B, max_q_len, T, Hq, Hkv, D, page, block_tables.shape[1],
                k_cache.shape[0], scale, window, status_tensor(q.device).data_ptr(),
                _stream(q.device)),
            "pxl_attn_prefill_tc",
        )
        _count()
        return out
    check(
        _lib.lib().pxl_attn_prefill(
            q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            block_tables.data_ptr(), cu_q.data_ptr(), ctx_lens.data_ptr(), out.data_ptr(),
            out.stride(0), _ptr(sinks), B, max_q_len, Hq, Hkv, D, page, block_tables.shape[1],
            k_cache.shape[0], scale, window, status_tensor(q.device).data_ptr(),
            _stream(q.device)),
        "pxl_attn_prefill",
    )
    _count()
    return out


# ------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, want_logprob: bool = False):
    B, V = logits.shape
    assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
    ids = torch.empty(B, dtype=torch.int32, device=logits.device)
    lp = torch.empty(B, dtype=torch.float32, device=logits.device) if want_logprob else None
    check(_lib.lib().pxl_argmax(logits.data_ptr(), int(logits.dtype == torch.bfloat16),
                                logits.stride(0), B, V, ids.data_ptr(), _ptr(lp),
                                status_tensor(logits.device).data_ptr(), _stream(logits.device)), "pxl_argmax")
    _count()
    return (ids, lp) if want_logprob else ids


def apply_penalties(logits: torch.Tensor, row_off: torch.Tensor, tok_ids: torch.Tensor, out_cnt: torch.Tensor,
                    rep: torch.Tensor, pres: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """Repetition / presence / frequency penalties in place on ``logits [B, V]`` (see ``csrc/sampler.cu``)."""
    B, V = logits.shape
    assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
    check(_lib.lib().pxl_apply_penalties(logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0), B, V,
                                         row_off.data_ptr(), tok_ids.data_ptr(), out_cnt.data_ptr(), rep.data_ptr(),
                                         pres.data_ptr(), freq.data_ptr(), status_tensor(logits.device).data_ptr(),
                                         _stream(logits.device)), "pxl_apply_penalties")
    _count()
    return logits


def sample(
    logits: torch.Tensor,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    min_p: torch.Tensor,
    uniform: torch.Tensor,
    want_prob: bool = False,
):
    B, V = logits.shape
    assert logits.stride(1) == 1
    ids = torch.empty(B, dtype=torch.int32, device=logits.device)
    pr = torch.empty(B, dtype=torch.float32, device=logits.device) if want_prob else None
    check(
        _lib.lib().pxl_sample(logits.data_ptr(), int(logits.dtype == torch.bfloat16),
                              logits.stride(0), B, V, temperature.data_ptr(), top_k.data_ptr(),
                              top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(),
                              ids.data_ptr(), _ptr(pr), status_tensor(logits.device).data_ptr(),
                              _stream(logits.device)),
        "pxl_sample",
    )
    _count()
    return (ids, pr) if want_prob else ids


# ------------------------------------------------------------------------------ MoE
def moe_route(logits: torch.Tensor, e_bias: Optional[torch.Tensor], k: int, mode: int = 0, renorm: bool = True,
              n_group: int = 1, topk_group: int = 1, routed_scale: float = 1.0):
    """Router logits ``[T, E]`` -> (expert ids int32 ``[T, k]``, weights fp32 ``[T, k]``)."""
    T, E = logits.shape
    assert logits.is_contiguous()
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    check(_lib.lib().pxl_moe_route(logits.data_ptr(), int(logits.dtype == torch.bfloat16), _ptr(e_bias), T, E, k,
                                   mode, int(renorm), n_group, topk_group, routed_scale, ids.data_ptr(),
                                   w.data_ptr(), _stream(logits.device)), "pxl_moe_route")
    _count()
    return ids, w


class MoEPlan:
    """Device-side expert-sorted layout of one batch (no host synchronisation)."""

    __slots__ = ("offsets", "mt_expert", "mt_row0", "mt_row_end", "num_mt", "pos_of", "src_tok", "max_mt",
                 "max_rows", "n_local")


def moe_align(ids: torch.Tensor, num_experts: int, e_lo: int = 0, e_hi: Optional[int] = None) -> MoEPlan:
    T, k = ids.shape
    e_hi = num_experts if e_hi is None else e_hi
    n_local = e_hi - e_lo
    dev = ids.device
    max_rows = T * k
    max_mt = (max_rows + 127) // 128 + n_local
    ints = torch.zeros(n_local * 2 + (n_local + 1) + 3 * max_mt + 1 + 2 * max_rows, dtype=torch.int32, device=dev)
    o = 0

    def take(n):
        nonlocal o
        v = ints[o:o + n]
        o += n
        return v

    counts, cursor, offsets = take(n_local), take(n_local), take(n_local + 1)
    p = MoEPlan()
    p.mt_expert, p.mt_row0, p.mt_row_end, p.num_mt = take(max_mt), take(max_mt), take(max_mt), take(1)
    p.pos_of, p.src_tok = take(max_rows), take(max_rows)
    p.offsets, p.max_mt, p.max_rows, p.n_local = offsets, max_mt, max_rows, n_local
    check(_lib.lib().pxl_moe_align(ids.data_ptr(), T, k, num_experts, e_lo, e_hi, counts.data_ptr(),
                                   offsets.data_ptr(), cursor.data_ptr(), p.mt_expert.data_ptr(),
                                   p.mt_row0.data_ptr(), p.mt_row_end.data_ptr(), p.num_mt.data_ptr(), max_mt,
                                   p.pos_of.data_ptr(), p.src_tok.data_ptr(), _stream(dev)), "pxl_moe_align")
    _count(4)
    return p


def moe_gather(x: torch.Tensor, plan: MoEPlan) -> torch.Tensor:
    H = x.shape[1]
    # one padding tile so that the last m-tile's TMA box stays inside the allocation
    xp = torch.empty((plan.max_rows + 128, H), dtype=x.dtype, device=x.device)
    check(_lib.lib().pxl_moe_gather(x.data_ptr(), plan.src_tok.data_ptr(), plan.offsets[plan.n_local:].data_ptr(),
                                    xp.data_ptr(), plan.max_rows, H, _stream(x.device)), "pxl_moe_gather")
    _count()
    return xp


def grouped_linear(a: torch.Tensor, w: torch.Tensor, plan: MoEPlan, num_local_experts: int,
                   epi: int = EPI_NONE, bn: int = 0, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [P, K]`` (expert-sorted rows) times stacked expert weights ``w [E*N, K]``."""
    P, K = a.shape
    N = w.shape[0] // num_local_experts
    n_out = N // 2 if epi == EPI_SILU_MUL else N
    out = torch.empty((P, n_out), dtype=a.dtype, device=a.device)
    check(_lib.lib().pxl_gemm_bf16_grouped(a.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(bias), P, num_local_experts, N, K,
                                           a.stride(0), w.stride(0), out.stride(0), plan.mt_expert.data_ptr(),
                                           plan.mt_row0.data_ptr(), plan.mt_row_end.data_ptr(),
                                           plan.num_mt.data_ptr(), plan.max_mt, epi, bn,
                                           status_tensor(a.device).data_ptr(), _stream(a.device)),
          "pxl_gemm_bf16_grouped")
    _count()
    return out


def moe_combine(y_perm: torch.Tensor, plan: MoEPlan, weights: torch.Tensor, base: Optional[torch.Tensor],
                T: int) -> torch.Tensor:
    k, H = weights.shape[1], y_perm.shape[1]
    out = torch.empty((T, H), dtype=y_perm.dtype, device=y_perm.device)
    check(_lib.lib().pxl_moe_combine(y_perm.data_ptr(), plan.pos_of.data_ptr(), weights.data_ptr(), _ptr(base),
                                     out.data_ptr(), T, k, H, _stream(y_perm.device)), "pxl_moe_combine")
    _count()
    return out


def moe_ffn(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
            num_experts: int, base: Optional[torch.Tensor] = None, act_mode: int = 0, limit: float = 0.0,
            b1: Optional[torch.Tensor] = None, b2: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``base + sum_j weights[:, j] * FFN_{ids[:, j]}(x)``.

    act_mode 0: SwiGLU fused into the first GEMM's epilogue; w1 ``[E * 2I, H]`` has gate/up rows
    interleaved per expert. act_mode 1: clipped ``swigluoai`` (GPT-OSS, MiniMax-M3): w1 holds
    ``[gate rows | up rows]`` per expert, optional expert biases b1 ``[E * 2I]`` / b2 ``[E * H]``.
    w2: ``[E * H, I]``."""
    plan = moe_align(ids, num_experts)
    xp = moe_gather(x, plan)
    if act_mode == 0:
        act = grouped_linear(xp, w1, plan, num_experts, epi=EPI_SILU_MUL)
    else:
        gu = grouped_linear(xp, w1, plan, num_experts, bias=b1)
        act = act_mul(gu, mode=act_mode, limit=limit)
    y = grouped_linear(act, w2, plan, num_experts, bias=b2)
    return moe_combine(y, plan, weights, base, x.shape[0])


def as_c_int_p(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


# ---------------------------------------------------------------------------- MLA / DSA
class _HeadPlan:
    """Static tile lists that run the grouped GEMM with attention heads in the role of experts:
    rows [h * Tpad, (h + 1) * Tpad) of a head-major matrix use weight block h."""

    __slots__ = ("mt_expert", "mt_row0", "mt_row_end", "num_mt", "max_mt")


_head_plans: dict = {}


def _head_plan(H: int, Tpad: int, device) -> _HeadPlan:
    key = (H, Tpad, device.index)
    p = _head_plans.get(key)
    if p is None:
        tiles = Tpad // 128
        h = torch.arange(H, dtype=torch.int32).repeat_interleave(tiles)
        i = torch.arange(tiles, dtype=torch.int32).repeat(H)
        p = _HeadPlan()
        p.mt_expert = h.to(device)
        p.mt_row0 = (h * Tpad + i * 128).to(device)
        p.mt_row_end = ((h + 1) * Tpad).to(device)
        p.num_mt = torch.tensor([H * tiles], dtype=torch.int32, device=device)
        p.max_mt = H * tiles
        _head_plans[key] = p
    return p


def _pad128(n: int) -> int:
    return max(128, (n + 127) // 128 * 128)


def mla_kv_prep(ckv, norm_w, cos_sin, positions, slot_mapping, cache, eps, latent: int):
    T = ckv.shape[0]
    rope = ckv.shape[1] - latent
    num_slots = cache.shape[0] * cache.shape[-2]
    check(_lib.lib().pxl_mla_kv_prep(ckv.data_ptr(), ckv.stride(0), norm_w.data_ptr(), cos_sin.data_ptr(),
                                     positions.data_ptr(), slot_mapping.data_ptr(), cache.data_ptr(), T, latent, rope,
                                     num_slots, eps, status_tensor(ckv.device).data_ptr(), _stream(ckv.device)),
          "pxl_mla_kv_prep")
    _count()


def mla_q_absorb(q, w_uk_s, cos_sin, positions, H: int, nope: int, latent: int):
    T = q.shape[0]
    rope = q.shape[1] // H - nope
    Tpad = _pad128(T)
    dev = q.device
    q_nope_hm = torch.zeros((H, Tpad, nope), dtype=q.dtype, device=dev) if Tpad != T else \
        torch.empty((H, Tpad, nope), dtype=q.dtype, device=dev)
    q_pe = torch.empty((T, H, rope), dtype=q.dtype, device=dev)
    check(_lib.lib().pxl_mla_q_prep(q.data_ptr(), q.stride(0), cos_sin.data_ptr(), positions.data_ptr(),
                                    q_nope_hm.data_ptr(), q_pe.data_ptr(), T, Tpad, H, nope, rope, _stream(dev)),
          "pxl_mla_q_prep")
    _count()
    plan = _head_plan(H, Tpad, dev)
    q_lat = grouped_linear(q_nope_hm.view(H * Tpad, nope), w_uk_s, plan, H)
    return q_lat.view(H, Tpad, latent), q_pe


def mla_attn(q_lat_hm, q_pe, cache, block_tables, cu_q, positions, scale, tok_begin: int, n_tok: int, topk=None,
             out=None):
    H, Tpad, L = q_lat_hm.shape
    if out is None:
        out = torch.zeros_like(q_lat_hm)
    if n_tok <= 0:
        return out
    B = block_tables.shape[0]
    check(_lib.lib().pxl_mla_attn(q_lat_hm.data_ptr(), q_pe.data_ptr(), cache.data_ptr(), block_tables.data_ptr(),
                                  _ptr(cu_q), positions.data_ptr(), _ptr(topk), out.data_ptr(), tok_begin, n_tok, Tpad,
                                  H, B, block_tables.shape[1], cache.shape[-2], L, q_pe.shape[-1],
                                  0 if topk is None else topk.shape[1], 0 if topk is None else topk.stride(0),
                                  float(scale), _stream(out.device)), "pxl_mla_attn")
    _count()
    return out


def mla_unabsorb(o_lat_hm, w_uv_s, T: int):
    H, Tpad, L = o_lat_hm.shape
    plan = _head_plan(H, Tpad, o_lat_hm.device)
    o = grouped_linear(o_lat_hm.view(H * Tpad, L), w_uv_s, plan, H)       # [H*Tpad, V]
    V = o.shape[1]
    return o.view(H, Tpad, V)[:, :T].transpose(0, 1).reshape(T, H * V)


def store_rows(src, slot_mapping, cache):
    T, D = src.shape
    num_slots = cache.numel() // D
    check(_lib.lib().pxl_store_rows(src.data_ptr(), src.stride(0), slot_mapping.data_ptr(), cache.data_ptr(), T, D,
                                    num_slots, status_tensor(src.device).data_ptr(), _stream(src.device)),
          "pxl_store_rows")
    _count()


def dsa_index_prep(q_idx, kv, k_off: int, w_off: int, ln_w, ln_b, ln_eps: float, cos_sin, positions, slot_mapping,
                   cache, w_scale: float, rope_dim: int):
    """Indexer pre-processing in one launch (``csrc/dsa.cu``): rotates ``q_idx [T, Hi, Di]`` in place, stores the
    normed + rotated index key of every token in ``cache`` and returns the scaled head weights ``[T, Hi]`` fp32."""
    T, Hi, Di = q_idx.shape
    assert q_idx.is_contiguous() and kv.stride(1) == 1 and kv.dtype == q_idx.dtype == torch.bfloat16
    w_out = torch.empty((T, Hi), dtype=torch.float32, device=q_idx.device)
    check(_lib.lib().pxl_dsa_index_prep(q_idx.data_ptr(), Hi * Di, kv.data_ptr(), kv.stride(0), k_off, w_off,
                                        ln_w.data_ptr(), _ptr(ln_b), ln_eps, cos_sin.data_ptr(), positions.data_ptr(),
                                        cos_sin.shape[0], slot_mapping.data_ptr(), cache.data_ptr(),
                                        cache.numel() // Di, w_out.data_ptr(), w_scale, T, Hi, Di, rope_dim,
                                        status_tensor(q_idx.device).data_ptr(), _stream(q_idx.device)),
          "pxl_dsa_index_prep")
    _count()
    return w_out


def dsa_index_scores(q_idx, w, index_cache, block_tables, cu_q, positions, max_ctx: int):
    T, Hi, Di = q_idx.shape
    ld = (max_ctx + 63) // 64 * 64
    scores = torch.empty((T, ld), dtype=torch.float32, device=q_idx.device)
    check(_lib.lib().pxl_dsa_index_scores(q_idx.data_ptr(), w.data_ptr(), index_cache.data_ptr(),
                                          block_tables.data_ptr(), _ptr(cu_q), positions.data_ptr(),
                                          scores.data_ptr(), ld, T, block_tables.shape[0], Hi, Di,
                                          block_tables.shape[1], index_cache.shape[-2], max_ctx,
                                          _stream(q_idx.device)), "pxl_dsa_index_scores")
    _count()
    return scores


def topk_select(scores, positions, k: int):
    T = scores.shape[0]
    out = torch.empty((T, k), dtype=torch.int32, device=scores.device)
    check(_lib.lib().pxl_topk_select(scores.data_ptr(), scores.stride(0), positions.data_ptr(), T, k, out.data_ptr(), k,
                                     _stream(scores.device)), "pxl_topk_select")
    _count()
    return out


# ---------------------------------------------------------------------------- block-scaled fp8
def quant_fp8_rows(x: torch.Tensor):
    """bf16 ``[T, K]`` -> (e4m3 ``[T, K]``, fp32 scales ``[T, K/128]``)."""
    T, K = x.shape
    q = torch.empty((T, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((T, K // 128), dtype=torch.float32, device=x.device)
    check(_lib.lib().pxl_quant_fp8_rows(x.data_ptr(), x.stride(0), q.data_ptr(), s.data_ptr(), T, K, _stream(x.device)),
          "pxl_quant_fp8_rows")
    _count()
    return q, s


def linear_fp8(x: torch.Tensor, wq: torch.Tensor, w_s64: torch.Tensor, residual: Optional[torch.Tensor] = None,
               epi: int = EPI_NONE) -> torch.Tensor:
    """``x [T, K]`` bf16 times block-scaled e4m3 weights ``wq [N, K]`` (scales ``[N/64, K/128]``)."""
    T, K = x.shape
    N = wq.shape[0]
    if residual is not None:
        epi = _lib.EPI_RESIDUAL
    xq, xs = quant_fp8_rows(x)
    n_out = N // 2 if epi == EPI_SILU_MUL else N
    out = torch.empty((T, n_out), dtype=torch.bfloat16, device=x.device)
    check(_lib.lib().pxl_gemm_fp8_block(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), w_s64.data_ptr(), out.data_ptr(),
                                        _ptr(residual), T, N, K, xq.stride(0), wq.stride(0), out.stride(0), epi,
                                        status_tensor(x.device).data_ptr(), _stream(x.device)), "pxl_gemm_fp8_block")
    _count()
    return out


def grouped_linear_fp8(a: torch.Tensor, wq: torch.Tensor, w_s64: torch.Tensor, plan, num_local_experts: int,
                       epi: int = EPI_NONE) -> torch.Tensor:
    """Expert-sorted rows ``a [P, K]`` bf16 times stacked e4m3 expert weights ``wq [E*N, K]``."""
    P, K = a.shape
    N = wq.shape[0] // num_local_experts
    aq, a_s = quant_fp8_rows(a)
    n_out = N // 2 if epi == EPI_SILU_MUL else N
    out = torch.empty((P, n_out), dtype=torch.bfloat16, device=a.device)
    check(_lib.lib().pxl_gemm_fp8_block_grouped(aq.data_ptr(), a_s.data_ptr(), wq.data_ptr(), w_s64.data_ptr(),
                                                out.data_ptr(), P, num_local_experts, N, K, aq.stride(0), wq.stride(0),
                                                out.stride(0), plan.mt_expert.data_ptr(), plan.mt_row0.data_ptr(),
                                                plan.mt_row_end.data_ptr(), plan.num_mt.data_ptr(), plan.max_mt, epi,
                                                status_tensor(a.device).data_ptr(), _stream(a.device)),
          "pxl_gemm_fp8_block_grouped")
    _count()
    return out


def moe_ffn_fp8(x, ids, weights, w1q, w1s, w2q, w2s, num_experts: int, base=None):
    """:func:`moe_ffn` with block-scaled e4m3 expert weights (activations quantised per 1x128 group)."""
    plan = moe_align(ids, num_experts)
    xp = moe_gather(x, plan)
    act = grouped_linear_fp8(xp, w1q, w1s, plan, num_experts, epi=EPI_SILU_MUL)
    y = grouped_linear_fp8(act, w2q, w2s, plan, num_experts)
    return moe_combine(y, plan, weights, base, x.shape[0])


# ---------------------------------------------------------------------------- gated delta net
def causal_conv1d_silu(x, w, bias, conv_state, seq_cu, seq_slots, positions):
    T, C = x.shape
    out = torch.empty((T, C), dtype=x.dtype, device=x.device)
    B = seq_slots.shape[0]
    check(_lib.lib().pxl_causal_conv1d_silu(x.data_ptr(), x.stride(0), w.data_ptr(), _ptr(bias), conv_state.data_ptr(),
                                            seq_cu.data_ptr(), seq_slots.data_ptr(), positions.data_ptr(),
                                            out.data_ptr(), out.stride(0), B, C, w.shape[1], _stream(x.device)),
          "pxl_causal_conv1d_silu")
    _count()
    return out


def gated_delta_rule(qkv, a, b, A_log, dt_bias, z, norm_w, rec_state, seq_cu, seq_slots, positions, Hk: int, Hv: int,
                     Dk: int, Dv: int, eps: float):
    T = qkv.shape[0]
    out = torch.empty((T, Hv * Dv), dtype=qkv.dtype, device=qkv.device)
    assert a.stride(0) == b.stride(0)
    check(_lib.lib().pxl_gated_delta_rule(qkv.data_ptr(), qkv.stride(0), a.data_ptr(), b.data_ptr(), a.stride(0),
                                          A_log.data_ptr(), dt_bias.data_ptr(), z.data_ptr(), z.stride(0),
                                          norm_w.data_ptr(), rec_state.data_ptr(), seq_cu.data_ptr(),
                                          seq_slots.data_ptr(), positions.data_ptr(), out.data_ptr(), out.stride(0),
                                          seq_slots.shape[0], Hk, Hv, Dk, Dv, eps, _stream(qkv.device)),
          "pxl_gated_delta_rule")
    _count()
    return out


def sigmoid_gate_mul(x, gate):
    T, N = x.shape
    out = torch.empty((T, N), dtype=x.dtype, device=x.device)
    check(_lib.lib().pxl_sigmoid_gate_mul(x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0), out.data_ptr(),
                                          out.stride(0), T, N, _stream(x.device)), "pxl_sigmoid_gate_mul")
    _count()
    return out


def gate_mul_grouped(x, gate, group: int, residual=None):
    """``(residual +) x * sigmoid(gate)`` with one gate value per ``group`` columns of ``x``."""
    T, N = x.shape
    x = x if x.stride(1) == 1 else x.contiguous()
    gate = gate if gate.stride(-1) == 1 else gate.contiguous()
    out = torch.empty((T, N), dtype=x.dtype, device=x.device)
    if residual is not None and residual.stride(1) != 1:
        residual = residual.contiguous()
    check(_lib.lib().pxl_gate_mul_grouped(x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0),
                                          _ptr(residual), residual.stride(0) if residual is not None else 0,
                                          out.data_ptr(), out.stride(0), T, N, int(group), _stream(x.device)),
          "pxl_gate_mul_grouped")
    _count()
    return out


def row_dot(x, w):
    """``x @ w`` for one weight row ``w [K]``: ``[T, 1]``."""
    T, K = x.shape
    x = x if x.stride(1) == 1 else x.contiguous()
    out = torch.empty((T, 1), dtype=x.dtype, device=x.device)
    check(_lib.lib().pxl_row_dot(x.data_ptr(), x.stride(0), w.contiguous().data_ptr(), out.data_ptr(), T, K,
                                 _stream(x.device)), "pxl_row_dot")
    _count()
    return out


# ---------------------------------------------------------------------------- block-sparse indexer (MSA)
def msa_block_scores(iq, index_cache, block_tables, cu_q, positions, max_ctx: int, sparse_block: int, scale: float):
    T, Hi, Di = iq.shape
    nb = (max_ctx + sparse_block - 1) // sparse_block
    scores = torch.empty((T, nb), dtype=torch.float32, device=iq.device)
    check(_lib.lib().pxl_msa_block_scores(iq.data_ptr(), index_cache.data_ptr(), block_tables.data_ptr(), _ptr(cu_q),
                                          positions.data_ptr(), scores.data_ptr(), nb, T, block_tables.shape[0], Hi, Di,
                                          block_tables.shape[1], index_cache.shape[-2], sparse_block, max_ctx,
                                          float(scale), _stream(iq.device)), "pxl_msa_block_scores")
    _count()
    return scores


def msa_select(scores, positions, block_tables, cu_q, page: int, sparse_block: int, topk: int, init_blocks: int,
               local_blocks: int):
    T = scores.shape[0]
    ppb = sparse_block // page
    v_tables = torch.zeros((T, topk * ppb), dtype=torch.int32, device=scores.device)
    v_ctx = torch.empty(T, dtype=torch.int32, device=scores.device)
    check(_lib.lib().pxl_msa_select(scores.data_ptr(), scores.stride(0), positions.data_ptr(), block_tables.data_ptr(),
                                    _ptr(cu_q), T, block_tables.shape[0], block_tables.shape[1], page, sparse_block, topk,
                                    init_blocks, local_blocks, v_tables.data_ptr(), v_tables.stride(0),
                                    v_ctx.data_ptr(), _stream(scores.device)), "pxl_msa_select")
    _count()
    return v_tables, v_ctx
