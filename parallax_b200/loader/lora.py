"""Batched LoRA: several adapters resident at once, each request of a batch using its own.

The reference loads PEFT adapters into its GPU backend and serves ``lora_path`` per request with a
segmented-GEMV kernel (``src/parallax/server/shard_loader.py:114-226``,
``src/parallax/server/executor/sglang_executor.py:249-333``, flags ``server_args.py:202-269``). Here the
low-rank update of a batch is two GROUPED tcgen05 GEMMs with the adapters in the role of experts: the rows
that use an adapter are gathered adapter by adapter, multiplied by the stacked ``A`` matrices, then by the
stacked ``B`` matrices, and added to the base projection's output with the adapter's scale. Rows without an
adapter are not touched.

Targets: ``q_proj / k_proj / v_proj`` (applied to the fused qkv projection as one update of rank 3r),
``o_proj`` and ``down_proj``. ``gate_proj`` / ``up_proj`` adapters cannot ride on the fused SiLU epilogue
and are only supported by merging an adapter into the weights at load time.

Ranks are padded to a multiple of 64 (one tile of the grouped GEMM), so the update costs a few per cent of
the base projection whatever the true rank.
"""

from __future__ import annotations

import json
import logging
import re
from collections import OrderedDict
from pathlib import Path
from typing import Optional

import torch

logger = logging.getLogger(__name__)

_KEY = re.compile(r"^(?:base_model\.model\.)?(?:model\.)?layers\.(\d+)\.(?:self_attn|mlp)\.(\w+)\.lora_([AB])"
                  r"(?:\.default)?\.weight$")
_KEY_MLX = re.compile(r"^(?:model\.)?(?:language_model\.)?(?:model\.)?layers\.(\d+)\.(?:self_attn|mlp)\.(\w+)\.lora_([ab])$")
TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "down_proj")


class LoRAAdapter:
    """One PEFT adapter on the host: ``{(layer, module): (A [r, in], B [out, r])}`` and its scale."""

    def __init__(self, name: str, rank: int, scaling: float, tensors: dict):
        self.name, self.rank, self.scaling, self.tensors = name, rank, scaling, tensors

    @classmethod
    def load(cls, path: str, name: Optional[str] = None) -> "LoRAAdapter":
        from safetensors.torch import load_file

        p = Path(path)
        cfg = json.loads((p / "adapter_config.json").read_text()) if (p / "adapter_config.json").exists() else {}
        mlx_file = p / "adapters.safetensors" if p.is_dir() else None
        if mlx_file is not None and mlx_file.exists() and not (p / "adapter_model.safetensors").exists():
            # the layout adapters are converted to for the reference's own backend
            # (src/parallax_utils/prepare_adapter.py): one file, ``...q_proj.lora_a [in, r]`` / ``lora_b [r, out]``,
            # ``lora_parameters: {rank, scale}`` with the scale applied as it stands
            lp = cfg.get("lora_parameters") or {}
            rank = int(lp.get("rank") or cfg.get("r") or 8)
            scaling = float(lp["scale"]) if "scale" in lp else float(cfg.get("lora_alpha", rank)) / rank
            raw = load_file(str(mlx_file))
            halves = {}
            for k, v in raw.items():
                m = _KEY_MLX.match(k)
                if m and m.group(2) in TARGETS + ("gate_proj", "up_proj"):
                    halves.setdefault((int(m.group(1)), m.group(2)), {})[m.group(3).upper()] = v.t().contiguous()
        else:
            rank = int(cfg.get("r") or cfg.get("lora_rank") or 8)
            scaling = float(cfg.get("lora_alpha", rank)) / rank
            raw = load_file(str(p / "adapter_model.safetensors" if p.is_dir() else p))
            halves = {}
            for k, v in raw.items():
                m = _KEY.match(k)
                if m and m.group(2) in TARGETS + ("gate_proj", "up_proj"):
                    halves.setdefault((int(m.group(1)), m.group(2)), {})[m.group(3)] = v
        unsupported = sorted({mod for (_l, mod) in halves if mod not in TARGETS})
        if unsupported:
            raise ValueError(f"adapter {path}: per-request serving covers {TARGETS}; it also has {unsupported} "
                             "(merge such an adapter into the weights at load time instead)")
        tensors = {k: (ab["A"].float(), ab["B"].float()) for k, ab in halves.items() if "A" in ab and "B" in ab}
        return cls(name or p.name, rank, scaling, tensors)


def _pad64(n: int) -> int:
    return (n + 63) // 64 * 64


class LoRAStack:
    """Device-side slots of one pipeline stage: for every local layer and fused target the ``A`` matrices of
    all slots stacked as ``[slots * R, in]`` and the ``B`` matrices as ``[slots * out, R]`` (R = padded rank),
    which is the weight layout of the grouped GEMM with one "expert" per slot."""

    def __init__(self, stage, max_slots: int, max_rank: int):
        cfg = stage.cfg
        self.stage = stage
        self.slots = max_slots
        self.device, self.dtype = stage.device, stage.dtype
        D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.r = max_rank
        self.dims = {"qkv": (H, (Hq + 2 * Hkv) * D, _pad64(3 * max_rank)), "o": (Hq * D, H, _pad64(max_rank)),
                     "down": (I, H, _pad64(max_rank))}
        self.q_out, self.kv_out = Hq * D, Hkv * D
        self.layers = []
        for lw in stage.layers:
            per = {}
            for tgt, (n_in, n_out, R) in self.dims.items():
                if tgt == "down" and lw.moe is not None:
                    continue
                per[tgt] = (torch.zeros((max_slots * R, n_in), dtype=self.dtype, device=self.device),
                            torch.zeros((max_slots * n_out, R), dtype=self.dtype, device=self.device))
            self.layers.append(per)
        self.scale = torch.zeros(max_slots, dtype=torch.float32, device=self.device)

    def load(self, slot: int, adapter: LoRAAdapter) -> None:
        if adapter.rank > self.r:
            raise ValueError(f"adapter {adapter.name} has rank {adapter.rank} > --max-lora-rank {self.r}")
        r = adapter.rank
        first = self.stage.start_layer
        for li, per in enumerate(self.layers):
            gl = first + li
            for tgt, (a_stack, b_stack) in per.items():
                n_in, n_out, R = self.dims[tgt]
                A = a_stack[slot * R:(slot + 1) * R]
                B = b_stack[slot * n_out:(slot + 1) * n_out]
                A.zero_()
                B.zero_()
                if tgt == "qkv":
                    row = 0
                    for j, (mod, width) in enumerate((("q_proj", self.q_out), ("k_proj", self.kv_out),
                                                      ("v_proj", self.kv_out))):
                        ab = adapter.tensors.get((gl, mod))
                        if ab is not None:
                            A[j * r:(j + 1) * r].copy_(ab[0])
                            B[row:row + width, j * r:(j + 1) * r].copy_(ab[1])
                        row += width
                else:
                    ab = adapter.tensors.get((gl, "o_proj" if tgt == "o" else "down_proj"))
                    if ab is not None:
                        A[:r].copy_(ab[0])
                        B[:, :r].copy_(ab[1])
        self.scale[slot] = adapter.scaling

    def apply(self, tgt: str, li: int, x: torch.Tensor, y: torch.Tensor, slot_of_row: torch.Tensor,
              plan=None) -> torch.Tensor:
        """``y + scale[slot] * (x A_slot^T) B_slot^T`` on the rows whose slot is >= 0 (``slot_of_row`` int32 [T])."""
        per = self.layers[li].get(tgt)
        if per is None:
            return y
        a_stack, b_stack = per
        _n_in, n_out, R = self.dims[tgt]
        if x.is_cuda:
            from parallax_b200.ops import cuda as cu

            plan = plan or cu.moe_align(slot_of_row.view(-1, 1), self.slots)
            xp = cu.moe_gather(x.contiguous(), plan)
            t = cu.grouped_linear(xp, a_stack, plan, self.slots, bn=64)
            d = cu.grouped_linear(t, b_stack, plan, self.slots)
            w = self.scale[slot_of_row.clamp_min(0).long()].view(-1, 1).contiguous()
            return cu.moe_combine(d, plan, w, y.contiguous(), x.shape[0])
        out = y.clone()
        for s in range(self.slots):
            rows = (slot_of_row == s).nonzero().flatten()
            if rows.numel():
                A = a_stack[s * R:(s + 1) * R].float()
                B = b_stack[s * n_out:(s + 1) * n_out].float()
                out[rows] = (out[rows].float() + float(self.scale[s]) * (x[rows].float() @ A.t()) @ B.t()).to(y.dtype)
        return out


class TPLoRAStack(LoRAStack):
    """Slots of a tensor-parallel stage whose residual stream is sharded by rows. The adapters are cut the way
    the base weights are: ``B`` of q/k/v keeps the rows of this rank's heads (``A`` whole), ``A`` of ``o_proj``
    and ``down_proj`` keeps the columns of this rank's heads / intermediate slice (``B`` whole). The rank-r
    intermediate is the only thing that crosses ranks: for q/k/v every rank projects its own rows and the
    ``[rows, r]`` pieces are all-gathered; for ``o_proj`` / ``down_proj`` the partial ``[T, r]`` products are
    reduce-scattered to the rows' owners, which add ``B`` times them to the projection's (already reduced)
    output. Plain matrix products per resident adapter: adapters are a small share of a step."""

    def __init__(self, stage, max_slots: int, max_rank: int):
        super().__init__(stage, max_slots, max_rank)
        cfg, tp = stage.cfg, stage.tp_size
        D, H, I = cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
        self.tp, self.tp_rank = tp, stage.tp_rank
        self.hq_l, self.hkv_l, self.i_l = stage.hq_l, stage.hkv_l, I // tp
        self.q_full, self.kv_full = self.q_out, self.kv_out
        self.q_out, self.kv_out = self.hq_l * D, self.hkv_l * D
        self.dims = {"qkv": (H, (self.hq_l + 2 * self.hkv_l) * D, _pad64(3 * max_rank)),
                     "o": (self.hq_l * D, H, _pad64(max_rank)), "down": (self.i_l, H, _pad64(max_rank))}
        for per in self.layers:
            for tgt in list(per):
                n_in, n_out, R = self.dims[tgt]
                per[tgt] = (torch.zeros((max_slots * R, n_in), dtype=self.dtype, device=self.device),
                            torch.zeros((max_slots * n_out, R), dtype=self.dtype, device=self.device))
        self.scale_host = [0.0] * max_slots

    def load(self, slot: int, adapter: LoRAAdapter) -> None:
        r, k = self.tp_rank, adapter.rank
        ql, kvl, il = self.q_out, self.kv_out, self.i_l
        cut = {}
        for (layer, mod), (A, B) in adapter.tensors.items():
            if mod == "q_proj":
                cut[(layer, mod)] = (A, B[r * ql:(r + 1) * ql])
            elif mod in ("k_proj", "v_proj"):
                cut[(layer, mod)] = (A, B[r * kvl:(r + 1) * kvl])
            elif mod == "o_proj":
                cut[(layer, mod)] = (A[:, r * ql:(r + 1) * ql], B)
            elif mod == "down_proj":
                cut[(layer, mod)] = (A[:, r * il:(r + 1) * il], B)
        super().load(slot, LoRAAdapter(adapter.name, k, adapter.scaling, cut))
        self.scale_host[slot] = float(adapter.scaling)

    def _index(self, fb, rp: int):
        """Per step: for every adapter slot in use the rows of the whole (padded) batch and this rank's own rows."""
        idx = fb.extras.get("_lora_tp_index")
        if idx is None or idx[0] != rp:
            host = fb.extras.get("lora_ids_host")
            if host is None:
                host = fb.extras["lora_ids"].cpu().numpy()
            import numpy as np

            full = np.full(rp * self.tp, -1, dtype=np.int64)
            full[:len(host)] = host
            mine = full[self.tp_rank * rp:(self.tp_rank + 1) * rp]
            per = {}
            for s in sorted(set(int(v) for v in full if v >= 0)):
                per[s] = (torch.from_numpy(np.nonzero(full == s)[0]).to(self.device),
                          torch.from_numpy(np.nonzero(mine == s)[0]).to(self.device))
            idx = fb.extras["_lora_tp_index"] = (rp, per)
        return idx[1]

    def apply_tp(self, tgt: str, li: int, x: torch.Tensor, y: torch.Tensor, fb, comm) -> torch.Tensor:
        """``tgt == "qkv"``: ``x`` are this rank's normalised rows ``[Rp, H]``, ``y`` the gathered batch's
        projection on this rank's heads ``[tp*Rp, cols]``. ``"o"`` / ``"down"``: ``x`` is the gathered batch on
        this rank's input slice ``[tp*Rp, in_local]``, ``y`` this rank's rows of the reduced output ``[Rp, H]``.
        Every rank of the group calls this for the same steps (the row -> adapter map is the whole batch's)."""
        per = self.layers[li].get(tgt)
        if per is None:
            return y
        a_stack, b_stack = per
        _n_in, n_out, R = self.dims[tgt]
        rp = x.shape[0] if tgt == "qkv" else y.shape[0]
        index = self._index(fb, rp)
        if not index:
            return y
        t = torch.zeros((x.shape[0], R), dtype=torch.float32, device=x.device)
        for s, (rows_all, rows_mine) in index.items():
            rows = rows_mine if tgt == "qkv" else rows_all
            if rows.numel():
                t[rows] = x[rows].float() @ a_stack[s * R:(s + 1) * R].float().t()
        t = comm.all_gather_rows(t) if tgt == "qkv" else comm.reduce_scatter_rows(t)
        y = y.clone() if not y.is_contiguous() else y
        for s, (rows_all, rows_mine) in index.items():
            rows = rows_all if tgt == "qkv" else rows_mine
            if rows.numel():
                d = t[rows] @ b_stack[s * n_out:(s + 1) * n_out].float().t()
                y[rows] = (y[rows].float() + self.scale_host[s] * d).to(y.dtype)
        return y


class LoRAManager:
    """Adapters by name: which are resident in which slot, least recently used ones make room. A slot that a
    running request uses is pinned."""

    def __init__(self, stacks: list[LoRAStack], max_loaded: int, paths: Optional[dict] = None, on_load=None):
        """``on_load(slot, name, path)``: called instead of loading into ``stacks`` - the multi-GPU engine
        sends the load to every rank with its next step plan."""
        self.stacks = stacks
        self.on_load = on_load
        self.max_loaded = max_loaded
        self.paths: dict[str, str] = dict(paths or {})
        self.slot_of: "OrderedDict[str, int]" = OrderedDict()       # resident adapters, least recently used first
        self.pins: dict[str, int] = {}
        self.free = list(range(max_loaded))

    def register(self, name: str, path: str) -> None:
        self.paths[name] = path

    def acquire(self, name_or_path: str) -> int:
        """Slot of the adapter (loading it if needed) with one more pin. Raises when every slot is pinned."""
        name = name_or_path
        if name not in self.paths:
            self.paths[name] = name_or_path          # a path used as its own name
        if name in self.slot_of:
            self.slot_of.move_to_end(name)
        else:
            if not self.free:
                victim = next((n for n in self.slot_of if not self.pins.get(n)), None)
                if victim is None:
                    raise RuntimeError("every LoRA slot is in use by a running request")
                self.free.append(self.slot_of.pop(victim))
            slot = self.free.pop()
            if self.on_load is not None:
                self.on_load(slot, name, self.paths[name])
            else:
                adapter = LoRAAdapter.load(self.paths[name], name)
                for st in self.stacks:
                    st.load(slot, adapter)
            self.slot_of[name] = slot
        self.pins[name] = self.pins.get(name, 0) + 1
        return self.slot_of[name]

    def release(self, name: str) -> None:
        if self.pins.get(name, 0) > 0:
            self.pins[name] -= 1


def parse_lora_paths(items) -> dict[str, str]:
    """``["name=path", "path", ...]`` -> ``{name: path}`` (a bare path is named after its last component)."""
    out = {}
    for it in items or []:
        name, _, path = it.partition("=")
        if not path:
            path, name = name, Path(name).name
        out[name] = path
    return out
