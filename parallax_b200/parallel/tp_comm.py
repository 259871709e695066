"""Tensor-parallel communication of a pipeline stage, behind one small interface.

The residual stream is sequence-sharded between the fused ops: rank r holds rows
``[r*Rp, (r+1)*Rp)`` of the (padded) token matrix. Two implementations:

* :class:`FusedTPComm` (B200): ``all_gather -> GEMM`` and ``GEMM -> reduce_scatter`` are single
  sm_100a kernels over NVLink peer memory (:mod:`parallax_b200.parallel.fused`).
* :class:`CollectiveTPComm`: library collectives of ``torch.distributed`` around plain
  ``ops.linear`` calls. With NCCL it is the *baseline* the fused kernels are measured against;
  with gloo it runs the sharding logic on CPU ranks in the tests.

The reference gets tensor parallelism from SGLang's column/row-parallel layers with an
all-reduce after o_proj / down_proj (``src/parallax/sglang/model_runner.py:134-179``) or from
``mx.distributed.all_sum`` on Apple (``src/parallax/models/qwen3.py:181-195``).
"""

from __future__ import annotations


import torch
import torch.distributed as dist

from parallax_b200 import ops


def padded_rows_per_rank(num_tokens: int, tp: int, align: int = 128) -> int:
    per = (num_tokens + tp - 1) // tp
    return max(align, (per + align - 1) // align * align)


class CollectiveTPComm:
    fused = False

    def __init__(self, group, tp: int, rank: int, align: int = 1):
        self.group, self.tp, self.rank, self.align = group, tp, rank, align

    def rows_per_rank(self, num_tokens: int) -> int:
        return padded_rows_per_rank(num_tokens, self.tp, self.align)

    def norm_ag_linear(self, h_shard, norm_w, eps, w, bias=None, epi: int = ops.EPI_NONE, w_offset: float = 0.0):
        """``linear(all_gather(rmsnorm(h_shard)), w)`` -> ``[tp*Rp, N_out]``."""
        xs = ops.rmsnorm(h_shard, norm_w, eps, w_offset=w_offset)
        full = torch.empty((xs.shape[0] * self.tp, xs.shape[1]), dtype=xs.dtype, device=xs.device)
        dist.all_gather_into_tensor(full, xs.contiguous(), group=self.group)
        if isinstance(w, tuple):      # block-scaled e4m3 weight with its scales
            return ops.linear_fp8(full, w[0], w[1], epi=epi)
        return ops.linear(full, w, bias=bias, epi=epi)

    def linear_rs(self, a, w, residual=None):
        """``reduce_scatter(a @ w^T) (+ residual)`` -> ``[Rp, N]``."""
        if isinstance(w, tuple):
            partial = ops.linear_fp8(a, w[0], w[1])
        else:
            partial = ops.linear(a, w, epi=ops.EPI_F32 if a.is_cuda else ops.EPI_NONE)
        partial = partial.float().contiguous()
        rp = a.shape[0] // self.tp
        if a.is_cuda:
            out = torch.empty((rp, partial.shape[1]), dtype=torch.float32, device=a.device)
            dist.reduce_scatter_tensor(out, partial, group=self.group)
        else:   # gloo has no reduce-scatter: all-reduce and keep the rows this rank owns
            dist.all_reduce(partial, group=self.group)
            out = partial[self.rank * rp:(self.rank + 1) * rp]
        if residual is not None:
            out = out + residual.float()
        return out.to(a.dtype)

    def moe_ffn(self, xn, n_valid: int, ids, weights, w1, w2, experts_per_rank: int, base=None):
        """Expert-parallel FFN on this rank's rows (experts sharded over the group)."""
        from parallax_b200.parallel.ep import ep_moe_ffn_nccl

        return ep_moe_ffn_nccl(self.group, xn, n_valid, ids, weights, w1, w2, experts_per_rank, base=base)

    def all_gather_rows(self, x_shard):
        full = torch.empty((x_shard.shape[0] * self.tp, x_shard.shape[1]), dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        return full

    def reduce_scatter_rows(self, x):
        """Sum ``[tp*Rp, n]`` over the group, keep this rank's ``Rp`` rows (fp32, small side products)."""
        x = x.float().contiguous()
        rp = x.shape[0] // self.tp
        if x.is_cuda:
            out = torch.empty((rp, x.shape[1]), dtype=torch.float32, device=x.device)
            dist.reduce_scatter_tensor(out, x, group=self.group)
            return out
        dist.all_reduce(x, group=self.group)
        return x[self.rank * rp:(self.rank + 1) * rp]

    def all_gather_cols(self, x):
        """Concatenate per-rank column blocks: ``[T, n] -> [T, tp*n]`` (vocab-parallel logits)."""
        parts = [torch.empty_like(x) for _ in range(self.tp)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


class FusedTPComm(CollectiveTPComm):
    fused = True

    def __init__(self, group, tp: int, rank: int, device, max_tokens: int, hidden: int, max_n: int, max_k: int):
        super().__init__(group, tp, rank, align=128)
        from parallax_b200.parallel.symm import TPWorkspace

        self._ep_ws = None
        self.ws = TPWorkspace(group, torch.device(device), tp, rank,
                              max_rows_per_rank=padded_rows_per_rank(max_tokens, tp), max_k=max(hidden, max_k),
                              max_n=max(hidden, max_n))

    def norm_ag_linear(self, h_shard, norm_w, eps, w, bias=None, epi: int = ops.EPI_NONE, w_offset: float = 0.0):
        from parallax_b200.parallel import fused

        token, xs = fused.gemm_ag_begin(self.ws, h_shard.shape[0], h_shard.shape[1])
        ops.rmsnorm(h_shard, norm_w, eps, w_offset=w_offset, out=xs)   # the norm writes straight into peer-visible memory
        return fused.gemm_ag(self.ws, token, w, bias=bias, epi=epi)

    def linear_rs(self, a, w, residual=None):
        from parallax_b200.parallel import fused

        return fused.gemm_rs(self.ws, a, w, residual=residual)

    def moe_ffn(self, xn, n_valid: int, ids, weights, w1, w2, experts_per_rank: int, base=None):
        from parallax_b200.parallel.ep import EPWorkspace, ep_moe_ffn

        if self._ep_ws is None:
            self._ep_ws = EPWorkspace(self.group, self.ws.device, self.tp, self.rank, self.ws.max_rows,
                                      ids.shape[1], xn.shape[1])
        out = torch.zeros_like(xn) if n_valid < xn.shape[0] else torch.empty_like(xn)
        return ep_moe_ffn(self._ep_ws, xn, n_valid, ids.contiguous(), weights.contiguous(), w1, w2, experts_per_rank,
                          base=base, out=out)
