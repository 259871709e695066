"""Python side of the native stage executor (``csrc/stage_exec.cu``): describes a dense GQA stage
once (weight and cache pointers per layer), then runs all of its layers for a step with a single
call into the kernel library. Used by :class:`parallax_b200.models.decoder.DecoderStage` on CUDA
devices when every layer of the stage is a plain dense layer."""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_int64, c_void_p

import torch

from parallax_b200.ops import _lib, cuda as cu
from parallax_b200.ops._lib import check


class _Layer(Structure):
    _fields_ = [(n, c_void_p) for n in ("ln1", "ln2", "w_qkv", "b_qkv", "q_norm", "k_norm", "w_o", "b_o", "w_gu",
                                        "w_down", "k_cache", "v_cache", "sinks")] + [("window", c_int), ("pad_", c_int)]


class _StageDesc(Structure):
    _fields_ = [(n, c_int) for n in ("H", "Hq", "Hkv", "D", "I", "rot_dim", "page", "n_layers")] + \
               [("num_blocks", c_int64), ("eps", c_float), ("norm_offset", c_float), ("scale", c_float),
                ("max_pos", c_int), ("cos_sin", c_void_p), ("layers", POINTER(_Layer))]


class _StepDesc(Structure):
    _fields_ = [(n, c_int) for n in ("T", "Tp", "Bp", "Bd", "p_max_q", "d_max_ctx", "p_max_blocks", "d_max_blocks")] + \
               [(n, c_void_p) for n in ("positions", "slots", "p_cu_q", "p_ctx", "p_bt", "d_ctx", "d_bt")]


class _Workspace(Structure):
    _fields_ = [(n, c_void_p) for n in ("xn", "qkv", "attn", "act", "h_a", "h_b", "decode")] + [("decode_floats", c_int64)]


def _p(t):
    return None if t is None else t.data_ptr()


class NativeDenseStage:
    def __init__(self, stage):
        cfg = stage.cfg
        self.stage = stage
        self.device = stage.device
        n = len(stage.layers)
        self._layers = (_Layer * n)()
        self._keep = []
        kc0 = stage.kv_caches[0].k
        for i, (lw, cache) in enumerate(zip(stage.layers, stage.kv_caches)):
            L = self._layers[i]
            for name in ("ln1", "ln2", "w_qkv", "b_qkv", "q_norm", "k_norm", "w_o", "b_o", "w_gu", "w_down", "sinks"):
                setattr(L, name, _p(getattr(lw, name)))
            L.k_cache, L.v_cache, L.window = cache.k.data_ptr(), cache.v.data_ptr(), int(lw.window or 0)
        d = _StageDesc()
        d.H, d.Hq, d.Hkv, d.D = cfg.hidden_size, cfg.num_attention_heads, kc0.shape[1], cfg.head_dim
        d.I, d.rot_dim, d.page, d.n_layers = stage.layers[0].w_down.shape[1], cfg.rot_dim, kc0.shape[2], n
        d.num_blocks, d.eps, d.norm_offset, d.scale = kc0.shape[0], cfg.rms_norm_eps, stage.norm_offset, stage.scale
        d.cos_sin, d.max_pos = stage.cos_sin.data_ptr(), int(stage.cos_sin.shape[0])
        d.layers = ctypes.cast(self._layers, POINTER(_Layer))
        self.desc = d
        self.qkv_n = (d.Hq + 2 * d.Hkv) * d.D
        self._cap = 0
        self._bufs = None
        self._ws = _Workspace()
        self._dec = None
        self._fn = _lib.bind("pxl_stage_forward_dense", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                         c_void_p, c_void_p])
        self._splits = _lib.lib().pxl_attn_decode_splits

    @staticmethod
    def supported(stage) -> bool:
        if stage.device.type != "cuda" or not stage.layers or not stage.kv_caches:
            return False
        if any(getattr(c, "k", None) is not None and c.k.dtype != stage.dtype for c in stage.kv_caches):
            return False            # e4m3 KV pages: the per-layer path picks the fp8 kernels
        if getattr(stage, "dense_act_mode", 0) or stage.cfg.qk_norm_full or any(getattr(lw, "w_g", None) is not None for lw in stage.layers):
            return False
        return all(lw.moe is None and lw.w_gu is not None and isinstance(lw.w_gu, torch.Tensor) for lw in stage.layers)

    def _ensure(self, T: int, Bd: int, d_max_ctx: int) -> None:
        d = self.desc
        if T > self._cap:
            cap = max(T, 256)
            dt, dev = self.stage.dtype, self.device
            self._bufs = [torch.empty((cap, n), dtype=dt, device=dev)
                          for n in (d.H, self.qkv_n, d.Hq * d.D, d.I, d.H, d.H)]
            w = self._ws
            w.xn, w.qkv, w.attn, w.act, w.h_a, w.h_b = [b.data_ptr() for b in self._bufs]
            self._cap = cap
        if Bd > 0:
            splits = self._splits(Bd, d.Hkv, d_max_ctx)
            need = Bd * d.Hq * splits * (d.D + 2) if splits > 1 else 0
            if self._dec is None or self._dec.numel() < need:
                self._dec = torch.empty(max(need, 1), dtype=torch.float32, device=self.device)
            self._ws.decode, self._ws.decode_floats = self._dec.data_ptr(), self._dec.numel()

    def forward(self, h_in: torch.Tensor, fb) -> torch.Tensor:
        T = fb.num_tokens
        self._ensure(T, fb.num_decode, fb.d_max_ctx)
        s = _StepDesc()
        s.T, s.Tp, s.Bp, s.Bd = T, fb.num_prefill_tokens, fb.num_prefill_seqs, fb.num_decode
        s.p_max_q, s.d_max_ctx = fb.p_max_q, fb.d_max_ctx
        s.positions, s.slots = fb.positions.data_ptr(), fb.slot_mapping.data_ptr()
        if s.Bp:
            s.p_cu_q, s.p_ctx, s.p_bt = fb.p_cu_q.data_ptr(), fb.p_ctx_lens.data_ptr(), fb.p_block_tables.data_ptr()
            s.p_max_blocks = fb.p_block_tables.shape[1]
        if s.Bd:
            s.d_ctx, s.d_bt, s.d_max_blocks = fb.d_ctx_lens.data_ptr(), fb.d_block_tables.data_ptr(), fb.d_block_tables.shape[1]
        out_ptr = c_void_p()
        n = c_int()
        assert h_in.is_contiguous()
        rc = self._fn(ctypes.addressof(self.desc), ctypes.addressof(s), ctypes.addressof(self._ws), h_in.data_ptr(),
                      ctypes.addressof(out_ptr), ctypes.addressof(n), cu.status_tensor(self.device).data_ptr(),
                      cu._stream(self.device))
        if rc >= 1000:      # debug mode of the executor: names the kernel that reported an error
            raise _lib.KernelError(f"stage executor: layer {(rc - 1000) // 16} op {(rc - 1000) % 16} reported a device error; "
                                   f"T={s.T} Tp={s.Tp} Bp={s.Bp} Bd={s.Bd} p_max_q={s.p_max_q} d_max_ctx={s.d_max_ctx} "
                                   f"p_max_blocks={s.p_max_blocks} d_max_blocks={s.d_max_blocks} "
                                   f"status={int(cu.status_tensor(self.device).item())}")
        check(rc, "pxl_stage_forward_dense")
        cu._count(n.value)
        buf = self._bufs[4] if out_ptr.value == self._ws.h_a else self._bufs[5]
        return buf[:T]
