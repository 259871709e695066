"""Expert-parallel MoE layer over NVLink peer memory (the kernels of ``csrc/moe_ep.cu`` plus the
scatter epilogue of the grouped tcgen05 GEMM).

Each rank of the group owns ``E / ep`` consecutive experts and a slice of the batch's token
rows. ``ep_moe_ffn`` routes nothing itself: it takes the rows, their expert ids and weights,
pushes every (row, slot) pair to the rank that owns the expert, runs the two grouped GEMMs
there and returns the expert outputs to the rank the row came from - the return trip is the
epilogue of the down projection, which stores each output row through a pointer into the source
rank's combine buffer. ``ep_moe_ffn_nccl`` is the library baseline (all-to-all of padded
buffers) that the benchmark compares against; it is not used for serving.

The reference runs with expert parallelism switched off
(``src/parallax/sglang/model_runner.py:394-395``).
"""

from __future__ import annotations

from ctypes import c_int, c_int64, c_uint32, c_void_p as P
from typing import Optional

import torch
import torch.distributed as dist

from parallax_b200.ops import _lib, cuda as cu
from parallax_b200.ops._lib import EPI_SILU_MUL, check
from parallax_b200.parallel.symm import SymmBuffer

_bound = {}


def _fn(name, argtypes):
    if name not in _bound:
        _bound[name] = _lib.bind(name, argtypes)
    return _bound[name]


def _dispatch_fn():
    return _fn("pxl_ep_dispatch", [P, c_int64, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P, P, P, P, P,
                                   c_uint32, P, P])


def _recv_ids_fn():
    return _fn("pxl_ep_recv_ids", [P, P, P, c_int, c_int, c_uint32, P, P, P])


def _row_ptrs_fn():
    return _fn("pxl_ep_row_ptrs", [P, P, P, c_int, c_int, c_int, P, P, c_int, P])


def _scatter_fn():
    return _fn("pxl_gemm_bf16_grouped_scatter", [P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, P, P, P, P, c_int,
                                                 P, P, c_int, c_int, c_uint32, P, P])


def _return_rows_fn():
    return _fn("pxl_ep_return_rows", [P, c_int64, P, P, c_int, c_int, P, P, c_int, c_int, c_uint32, P])


def _combine_fn():
    return _fn("pxl_ep_combine", [P, P, P, c_int64, P, c_int64, P, c_int, c_uint32, c_int, c_int, c_int, P, P])


class EPWorkspace:
    """Symmetric receive / combine buffers of one expert-parallel group."""

    def __init__(self, group, device: torch.device, ep: int, rank: int, max_rows_per_rank: int, top_k: int,
                 hidden: int):
        self.group, self.device, self.ep, self.rank = group, device, ep, rank
        self.max_rows, self.k, self.H = max_rows_per_rank, top_k, hidden
        self.cap = max_rows_per_rank * top_k          # worst case: every pair of one source lands on one rank
        n_recv = ep * self.cap
        self.off_recv_x = 0
        self.off_comb = self.off_recv_x + n_recv * hidden * 2
        self.off_meta = self.off_comb + self.cap * hidden * 2
        self.off_cnt = self.off_meta + n_recv * 8
        self.off_dflag = self.off_cnt + 64
        self.off_rflag = self.off_dflag + 64
        total = self.off_rflag + 64
        self.buf = SymmBuffer(total, group, device)
        self.recv_x = self.buf.view(self.off_recv_x, (n_recv, hidden), torch.bfloat16)
        self.comb = self.buf.view(self.off_comb, (self.cap, hidden), torch.bfloat16)
        self.recv_meta = self.buf.view(self.off_meta, (n_recv, 2), torch.int32)
        self.recv_cnt = self.buf.view(self.off_cnt, (16,), torch.int32)
        self.disp_flag = self.buf.view(self.off_dflag, (16,), torch.int32)
        self.ret_flag = self.buf.view(self.off_rflag, (16,), torch.int32)
        # local scratch
        self.cursor = torch.zeros(16, dtype=torch.int32, device=device)
        self.counters = torch.zeros(4, dtype=torch.int32, device=device)
        self.ids_local = torch.empty(n_recv, dtype=torch.int32, device=device)
        self.row_ptrs = torch.zeros(n_recv + 256, dtype=torch.int64, device=device)
        self.epoch = 0
        self._p = {name: self.buf.ptr_array(off) for name, off in
                   (("recv_x", self.off_recv_x), ("comb", self.off_comb), ("meta", self.off_meta),
                    ("cnt", self.off_cnt), ("dflag", self.off_dflag), ("rflag", self.off_rflag))}


def ep_moe_ffn(ws: EPWorkspace, x: torch.Tensor, n_valid: int, ids: torch.Tensor, weights: torch.Tensor,
               w1, w2, experts_per_rank: int, base: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, max_rows: Optional[int] = None, fp8: Optional[dict] = None,
               act_mode: int = 0, limit: float = 0.0, b1=None, b2=None) -> torch.Tensor:
    """``out[:n_valid] = base + sum_j weights[:, j] * FFN_{ids[:, j]}(x)`` for this rank's rows.

    x ``[rows, H]``, ids/weights ``[rows, k]`` (global expert ids); w1 ``[E_local * 2I, H]``
    (gate/up interleaved), w2 ``[E_local * H, I]`` hold this rank's experts only.

    ``max_rows``: an upper bound of ``n_valid`` over ALL ranks of the group for this call (every rank must
    pass the same value); it sizes the receive regions of the call, so a decode step does not scan the
    regions of the largest prefill batch. ``fp8``: ``{"w1": (q, scales), "w2": (q, scales)}`` block-scaled
    e4m3 expert weights; the expert outputs then return through a copy kernel instead of the GEMM epilogue.
    ``act_mode`` 1: clipped ``swigluoai`` experts with biases (the activation is its own kernel)."""
    dev = x.device
    H, k = ws.H, ws.k
    assert x.shape[1] == H and ids.shape[1] == k and n_valid <= ws.max_rows
    cap = ws.cap if max_rows is None else max(min(max_rows, ws.max_rows), 1) * k
    assert n_valid * k <= cap
    n_recv = ws.ep * cap
    ws.epoch += 1
    epoch = ws.epoch
    st = cu.status_tensor(dev).data_ptr()
    stream = cu._stream(dev)
    check(_dispatch_fn()(x.data_ptr(), x.stride(0), ids.data_ptr(), n_valid, k, H, experts_per_rank, cap, ws.rank,
                         ws.ep, ws._p["recv_x"], ws._p["meta"], ws._p["cnt"], ws._p["dflag"], ws.cursor.data_ptr(),
                         ws.counters[0:].data_ptr(), epoch, st, stream), "pxl_ep_dispatch")
    ids_local = ws.ids_local[:n_recv]
    check(_recv_ids_fn()(ws.recv_meta.data_ptr(), ws.recv_cnt.data_ptr(), ws.disp_flag.data_ptr(), ws.ep, cap,
                         epoch, ids_local.data_ptr(), st, stream), "pxl_ep_recv_ids")
    cu._count(2)
    plan = cu.moe_align(ids_local.view(-1, 1), experts_per_rank)
    xp = cu.moe_gather(ws.recv_x, plan)
    n_rows_dev = plan.offsets[plan.n_local:]
    check(_row_ptrs_fn()(plan.src_tok.data_ptr(), n_rows_dev.data_ptr(), ws.recv_meta.data_ptr(), cap, H, ws.ep,
                         ws._p["comb"], ws.row_ptrs.data_ptr(), plan.max_rows, stream), "pxl_ep_row_ptrs")
    if fp8 is None and act_mode == 0:
        act = cu.grouped_linear(xp, w1, plan, experts_per_rank, epi=EPI_SILU_MUL)
        N = w2.shape[0] // experts_per_rank
        check(_scatter_fn()(act.data_ptr(), w2.data_ptr(), ws.row_ptrs.data_ptr(), act.shape[0], experts_per_rank, N,
                            act.shape[1], act.stride(0), w2.stride(0), plan.mt_expert.data_ptr(),
                            plan.mt_row0.data_ptr(), plan.mt_row_end.data_ptr(), plan.num_mt.data_ptr(), plan.max_mt,
                            ws._p["rflag"], ws.counters[1:].data_ptr(), ws.rank, ws.ep, epoch, st, stream),
              "pxl_gemm_bf16_grouped_scatter")
    else:
        if fp8 is not None:
            act = cu.grouped_linear_fp8(xp, *fp8["w1"], plan, experts_per_rank, epi=EPI_SILU_MUL)
            y = cu.grouped_linear_fp8(act, *fp8["w2"], plan, experts_per_rank)
        else:
            gu = cu.grouped_linear(xp, w1, plan, experts_per_rank, bias=b1)
            act = cu.act_mul(gu, mode=act_mode, limit=limit)
            y = cu.grouped_linear(act, w2, plan, experts_per_rank, bias=b2)
        check(_return_rows_fn()(y.data_ptr(), y.stride(0), ws.row_ptrs.data_ptr(), n_rows_dev.data_ptr(), plan.max_rows,
                                H, ws._p["rflag"], ws.counters[1:].data_ptr(), ws.rank, ws.ep, epoch, stream),
              "pxl_ep_return_rows")
    if out is None:
        out = torch.empty_like(x)
    check(_combine_fn()(ws.comb.data_ptr(), weights.data_ptr(), None if base is None else base.data_ptr(),
                        0 if base is None else base.stride(0), out.data_ptr(), out.stride(0), ws.ret_flag.data_ptr(),
                        ws.ep, epoch, n_valid, k, H, st, stream), "pxl_ep_combine")
    cu._count(3)
    return out


def ep_moe_ffn_nccl(group, x: torch.Tensor, n_valid: int, ids: torch.Tensor, weights: torch.Tensor, w1, w2,
                    experts_per_rank: int, base: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Library baseline with the same sharding: all-gather rows and routing, every rank applies
    its own experts to all rows (others masked out), reduce-scatter of the partial sums."""
    ep = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows, H = x.shape
    k = ids.shape[1]
    xa = torch.empty((ep * rows, H), dtype=x.dtype, device=x.device)
    ia = torch.empty((ep * rows, k), dtype=ids.dtype, device=x.device)
    wa = torch.empty((ep * rows, k), dtype=weights.dtype, device=x.device)
    valid = torch.zeros(rows, dtype=torch.int32, device=x.device)
    valid[:n_valid] = 1
    va = torch.empty(ep * rows, dtype=torch.int32, device=x.device)
    dist.all_gather_into_tensor(xa, x.contiguous(), group=group)
    dist.all_gather_into_tensor(ia, ids.contiguous(), group=group)
    dist.all_gather_into_tensor(wa, weights.contiguous(), group=group)
    dist.all_gather_into_tensor(va, valid, group=group)
    lo = rank * experts_per_rank
    local = (ia >= lo) & (ia < lo + experts_per_rank) & (va[:, None] > 0)
    ids_l = torch.where(local, ia - lo, torch.full_like(ia, -1))
    from parallax_b200 import ops

    if x.is_cuda:
        plan = cu.moe_align(ids_l.contiguous(), experts_per_rank)
        xp = cu.moe_gather(xa, plan)
        act = cu.grouped_linear(xp, w1, plan, experts_per_rank, epi=EPI_SILU_MUL)
        y = cu.grouped_linear(act, w2, plan, experts_per_rank)
        part = cu.moe_combine(y, plan, wa.float().contiguous(), None, ep * rows).float()
    else:
        wl = torch.where(local, wa.float(), torch.zeros_like(wa, dtype=torch.float32))
        part = ops.reference.moe_ffn(xa, ids_l.clamp_min(0), wl, w1, w2, experts_per_rank).float()
    if x.is_cuda:
        outp = torch.empty((rows, H), dtype=torch.float32, device=x.device)
        dist.reduce_scatter_tensor(outp, part.contiguous(), group=group)
    else:
        dist.all_reduce(part, group=group)
        outp = part[rank * rows:(rank + 1) * rows]
    if base is not None:
        outp = outp + base.float()
    return outp.to(x.dtype)


def ep_moe_ffn_ragged(group, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, local_ffn, experts_per_rank: int,
                      base: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Library formulation for ranks that hold DIFFERENT numbers of rows (attention data-parallel):
    rows, routing and weights are padded to the largest rank and all-gathered, every rank applies its own
    experts to all rows (``local_ffn(x_all, local_ids, local_weights) -> [rows, H]`` with weight 0 on the
    pairs of other ranks), the partial sums are all-reduced and each rank keeps its own rows. Used on CPU
    ranks (gloo) and as the baseline; serving on GPUs takes :func:`ep_moe_ffn`."""
    ep = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T, H = x.shape
    k = ids.shape[1]
    sizes = torch.zeros(ep, dtype=torch.int64, device=x.device)
    sizes[rank] = T
    dist.all_reduce(sizes, group=group)
    t_max = max(int(sizes.max()), 1)

    def padded(t, fill=0):
        out = t.new_full((t_max,) + tuple(t.shape[1:]), fill)
        out[:T] = t
        return out

    xa = torch.empty((ep * t_max, H), dtype=x.dtype, device=x.device)
    ia = torch.empty((ep * t_max, k), dtype=ids.dtype, device=x.device)
    wa = torch.empty((ep * t_max, k), dtype=weights.dtype, device=x.device)
    dist.all_gather_into_tensor(xa, padded(x), group=group)
    dist.all_gather_into_tensor(ia, padded(ids, -1), group=group)
    dist.all_gather_into_tensor(wa, padded(weights), group=group)
    lo = rank * experts_per_rank
    local = (ia >= lo) & (ia < lo + experts_per_rank)
    ids_l = torch.where(local, ia - lo, torch.zeros_like(ia))
    w_l = torch.where(local, wa.float(), torch.zeros_like(wa, dtype=torch.float32))
    part = local_ffn(xa, ids_l.to(torch.int32), w_l).float()
    dist.all_reduce(part, group=group)
    out = part[rank * t_max:rank * t_max + T]
    if base is not None:
        out = out + base.float()
    return out.to(x.dtype)


class EPComm:
    """Expert parallelism for a group whose ranks run attention data-parallel: every rank brings its own
    token rows (any number, also none), experts are sharded over the group. On B200 the exchange is the
    peer-memory dispatch / combine of :func:`ep_moe_ffn`; on CPU ranks the library formulation."""

    def __init__(self, group, ep: int, rank: int, device, max_rows: int, fused: Optional[bool] = None):
        self.group, self.ep, self.rank = group, ep, rank
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.fused = (self.device.type == "cuda") if fused is None else fused
        self._ws: Optional[EPWorkspace] = None
        self.step_max_rows: Optional[int] = None     # set by the engine per step: largest row count over the ranks

    def _warm_up(self, moe, dtype) -> None:
        """First use: one exchange without rows, between two host barriers. The kernels of an exchange wait
        for their peers on the device for at most a second or so; loading the kernels and allocating their
        scratch for the first time can take a rank longer than that, so this first round is run with every
        rank known to be at the same point, and serving starts with everything resident."""
        H, k = self._ws.H, self._ws.k
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        x0 = torch.empty((0, H), dtype=dtype, device=self.device)
        ep_moe_ffn(self._ws, x0, 0, torch.empty((0, k), dtype=torch.int32, device=self.device),
                   torch.empty((0, k), dtype=torch.float32, device=self.device), moe.w1, moe.w2, moe.experts_per_rank,
                   max_rows=1, fp8=moe.fp8, act_mode=moe.act_mode, limit=moe.limit, b1=moe.b1, b2=moe.b2)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def moe_ffn(self, moe, xn: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, base=None) -> torch.Tensor:
        """``base + MoE(xn)`` for this rank's rows; ``moe`` is the layer's (expert-sharded) MoEWeights."""
        from parallax_b200 import ops

        epr = moe.experts_per_rank
        if not self.fused:
            def local_ffn(xa, ids_l, w_l):
                if moe.fp8 is not None:
                    return ops.moe_ffn_fp8(xa, ids_l, w_l, *moe.fp8["w1"], *moe.fp8["w2"], epr)
                if moe.act_mode:
                    return ops.moe_ffn(xa, ids_l, w_l, moe.w1, moe.w2, epr, act_mode=moe.act_mode, limit=moe.limit,
                                       b1=moe.b1, b2=moe.b2)
                return ops.moe_ffn(xa, ids_l, w_l, moe.w1, moe.w2, epr)

            return ep_moe_ffn_ragged(self.group, xn, ids, weights, local_ffn, epr, base=base)
        if self._ws is None:
            self._ws = EPWorkspace(self.group, self.device, self.ep, self.rank, self.max_rows, ids.shape[1], xn.shape[1])
            self._warm_up(moe, xn.dtype)
        return ep_moe_ffn(self._ws, xn, xn.shape[0], ids.contiguous(), weights.contiguous(), moe.w1, moe.w2, epr,
                          base=base, max_rows=self.step_max_rows, fp8=moe.fp8, act_mode=moe.act_mode,
                          limit=moe.limit, b1=moe.b1, b2=moe.b2)
