"""Symmetric (peer-mapped) device memory for the fused tensor-/expert-parallel kernels.

Every rank of a group allocates the same buffer; after the rendezvous each rank knows the
device address of every peer's copy (NVLink peer mappings) and, when the fabric supports it,
a multicast address that targets all copies at once (NVLS). Allocation and address exchange
use ``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged over the process
group's store); everything that runs on the hot path - the loads, stores, flags and waits -
is in the kernels of ``csrc/gemm_tcgen05.cu`` and ``csrc/moe_ep.cu``.

``TPWorkspace`` bundles the buffers the fused GEMM->reduce-scatter and all-gather->GEMM need
(two alternating sets, so that a buffer is never rewritten while a slow peer may still read
the previous use) and hands out monotonically increasing epochs for their flags.
"""

from __future__ import annotations

import ctypes

import torch


class SymmBuffer:
    def __init__(self, nbytes: int, group, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.nbytes = (nbytes + 255) // 256 * 256
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.local, group=group)
        self.local.zero_()
        self.world_size = self.handle.world_size
        self.rank = self.handle.rank
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr) if self.handle.has_multicast_support(
                device.type, device.index) else 0
        except Exception:
            self.multicast_ptr = 0
        torch.cuda.synchronize(device)
        self.handle.barrier()

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = int(torch.tensor(shape).prod()) * torch.empty(0, dtype=dtype).element_size()
        return self.local[offset:offset + n].view(dtype).view(*shape)

    def ptr_array(self, offset: int = 0):
        arr = (ctypes.c_void_p * 8)()
        for i, p in enumerate(self.ptrs):
            arr[i] = p + offset
        return arr

    def barrier(self) -> None:
        self.handle.barrier()


class TPWorkspace:
    """Buffers of one tensor-parallel group sized for ``max_rows_per_rank`` token rows."""

    def __init__(self, group, device: torch.device, tp: int, rank: int, max_rows_per_rank: int, max_k: int,
                 max_n: int, num_sets: int = 2):
        self.tp, self.rank, self.device = tp, rank, device
        self.max_rows = max_rows_per_rank
        self.max_k, self.max_n = max_k, max_n
        rows_all = tp * max_rows_per_rank
        self.x_bytes = rows_all * max_k * 2                    # gathered activations
        self.stage_bytes = tp * max_rows_per_rank * max_n * 2   # reduce-scatter staging
        max_tiles = tp * (max_rows_per_rank // 128) * ((max_n + 63) // 64)
        self.flag_bytes = (max_tiles + tp + 64) * 4
        per_set = self.x_bytes + self.stage_bytes + 2 * self.flag_bytes
        self.per_set = (per_set + 255) // 256 * 256
        self.buf = SymmBuffer(self.per_set * num_sets, group, device)
        self.num_sets = num_sets
        self._use = 0
        self._epoch = [0] * num_sets
        # local (non-symmetric) flags of the all-gather: 16 chunk flags per 128-row tile
        self.tile_flags = torch.zeros((num_sets, (rows_all // 128 + 8) * 16), dtype=torch.int32, device=device)

    def next_set(self) -> tuple[int, int]:
        """(set index, epoch) for the next fused op."""
        s = self._use
        self._use = (self._use + 1) % self.num_sets
        self._epoch[s] += 1
        return s, self._epoch[s]

    # offsets inside a set
    def x_off(self, s: int) -> int:
        return s * self.per_set

    def stage_off(self, s: int) -> int:
        return s * self.per_set + self.x_bytes

    def rs_flag_off(self, s: int) -> int:
        return s * self.per_set + self.x_bytes + self.stage_bytes

    def ag_flag_off(self, s: int) -> int:
        return self.rs_flag_off(s) + self.flag_bytes

    def x_full(self, s: int, rows_per_rank: int, k: int) -> torch.Tensor:
        """This rank's copy of the gathered matrix ``[tp * rows_per_rank, k]`` of set ``s``."""
        return self.buf.view(self.x_off(s), (self.tp * rows_per_rank, k), torch.bfloat16)

    def x_shard(self, s: int, rows_per_rank: int, k: int) -> torch.Tensor:
        return self.x_full(s, rows_per_rank, k)[self.rank * rows_per_rank:(self.rank + 1) * rows_per_rank]
