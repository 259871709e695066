"""Plain-PyTorch restatement of every op (the correctness oracle and the CPU path).

These functions accept the same arguments as :mod:`parallax_b200.ops.cuda`, run on any
device and dtype, and compute in fp32 internally. They restate the arithmetic of the
reference's Metal compute kernels (which have no CPU implementation of their own):
single-query paged attention with sliding window and sinks
(``src/parallax_extensions/kernels/paged_attention/paged_attention.metal:794-1234``), the
cache scatter (``.../reshape_and_cache/reshape_and_cache.metal:32-96``), and the sampler
(``src/parallax/server/sampling/sampler.py:65-120``).
"""

from __future__ import annotations

import math

import torch

EPI_NONE, EPI_RESIDUAL, EPI_SILU_MUL, EPI_F32 = 0, 1, 2, 3


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Arrange gate/up weight rows for the fused SiLU-mul GEMM epilogue.

    Rows are grouped in blocks of 128: 64 gate rows followed by the 64 up rows of the same
    output columns.
    """
    I, K = w_gate.shape
    h = 64
    assert I % h == 0
    g = w_gate.reshape(I // h, h, K)
    u = w_up.reshape(I // h, h, K)
    return torch.cat([g, u], dim=1).reshape(2 * I, K).contiguous()


def linear(x, w, bias=None, residual=None, epi: int = EPI_NONE, out=None, bn: int = 128):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
        epi = EPI_RESIDUAL
    if epi == EPI_SILU_MUL:
        N = w.shape[0]
        h = 64
        yb = y.reshape(y.shape[0], N // 128, 2, h)
        y = (torch.nn.functional.silu(yb[:, :, 0]) * yb[:, :, 1]).reshape(y.shape[0], N // 2)
    res = y if epi == EPI_F32 else y.to(x.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def rmsnorm(x, weight, eps, residual=None, w_offset: float = 0.0, out=None):
    xf = x.float()
    if residual is not None:
        s = (xf + residual.float()).to(x.dtype)
        residual.copy_(s)
        xf = s.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * inv * (weight.float() + w_offset)).to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def build_cos_sin(max_pos: int, rot_dim: int, base: float, device=None, inv_freq=None,
                  attention_factor: float = 1.0) -> torch.Tensor:
    """fp32 table ``[max_pos, rot_dim]``: cos in the first half of each row, sin in the second."""
    if inv_freq is None:
        inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float64)
    freqs = torch.outer(t, inv_freq.double())
    tab = torch.cat([freqs.cos(), freqs.sin()], dim=-1) * attention_factor
    return tab.float().to(device) if device is not None else tab.float()


_E4M3_MAX = 448.0


def _scatter_cache(cache, x, slot_mapping, scale: float = 1.0):
    # cache [blocks, H, page, D]; x [T, H, D]. An e4m3 cache stores x / scale, saturating.
    page = cache.shape[2]
    valid = slot_mapping >= 0
    if not bool(valid.any()):
        return
    slots = slot_mapping[valid]
    blk = slots // page
    off = slots % page
    if cache.dtype == torch.float8_e4m3fn:
        val = (x[valid].float() / scale).clamp(-_E4M3_MAX, _E4M3_MAX).to(cache.dtype)
        cache.view(torch.uint8)[blk, :, off, :] = val.view(torch.uint8)
    else:
        cache[blk, :, off, :] = x[valid].to(cache.dtype)


def qk_norm_rope_cache(qkv, q_norm_w, k_norm_w, cos_sin, positions, slot_mapping, k_cache,
                       v_cache, num_q_heads, num_kv_heads, head_dim, rot_dim, eps=1e-6,
                       norm_w_offset: float = 0.0, kv_scale=(1.0, 1.0)):
    T = qkv.shape[0]
    Hq, Hkv, D = num_q_heads, num_kv_heads, head_dim
    x = qkv.view(T, Hq + 2 * Hkv, D)
    q, k, v = x[:, :Hq], x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]

    def norm(t, w):
        if w is None:
            return t.float()
        tf = t.float()
        inv = torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + eps)
        return (tf * inv * (w.float() + norm_w_offset)).to(qkv.dtype).float()

    def rope(t):
        if cos_sin is None or rot_dim == 0:
            return t
        half = rot_dim // 2
        cs = cos_sin[positions.long()].float()  # [T, rot_dim]
        cos, sin = cs[:, None, :half], cs[:, None, half:]
        x1, x2 = t[..., :half], t[..., half:rot_dim]
        out = t.clone()
        out[..., :half] = x1 * cos - x2 * sin
        out[..., half:rot_dim] = x2 * cos + x1 * sin
        return out

    qn = rope(norm(q, q_norm_w)).to(qkv.dtype)
    kn = rope(norm(k, k_norm_w)).to(qkv.dtype)
    q.copy_(qn)
    if k_cache is not None and slot_mapping is not None:
        _scatter_cache(k_cache, kn, slot_mapping, kv_scale[0])
        _scatter_cache(v_cache, v, slot_mapping, kv_scale[1])
    else:
        k.copy_(kn)


def reshape_and_cache(k, v, slot_mapping, k_cache, v_cache, kv_scale=(1.0, 1.0)):
    if k is not None and k_cache is not None:
        _scatter_cache(k_cache, k, slot_mapping, kv_scale[0])
    if v is not None and v_cache is not None:
        _scatter_cache(v_cache, v, slot_mapping, kv_scale[1])


def act_mul(x, mode: int = 0, limit: float = 7.0):
    I = x.shape[-1] // 2
    g, u = x[..., :I].float(), x[..., I:].float()
    if mode == 0:
        y = torch.nn.functional.silu(g) * u
    elif mode == 1:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
        y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    else:
        y = torch.nn.functional.gelu(g, approximate="tanh") * u
    return y.to(x.dtype)


def gather_rows(table, ids, out=None):
    y = table[ids.long()]
    if out is not None:
        out.copy_(y)
        return out
    return y


def add_inplace(y, x):
    y.add_(x)
    return y


def _gather_kv(cache, block_table, n, scale: float = 1.0):
    # cache [blocks, H, page, D] -> [H, n, D]; an e4m3 cache is widened and multiplied by its scale
    page = cache.shape[2]
    nb = (n + page - 1) // page
    if cache.dtype == torch.float8_e4m3fn:
        blocks = cache.view(torch.uint8)[block_table[:nb].long()].view(torch.float8_e4m3fn).float() * scale
    else:
        blocks = cache[block_table[:nb].long()]  # [nb, H, page, D]
    return blocks.permute(1, 0, 2, 3).reshape(cache.shape[1], nb * page, cache.shape[3])[:, :n]


def _attend(q, k, v, scale, q_pos, window, sinks):
    # q [Lq, Hq, D]; k, v [Hkv, Lk, D]; q_pos [Lq] absolute positions of the queries
    Lq, Hq, D = q.shape
    Hkv, Lk, _ = k.shape
    G = Hq // Hkv
    qf = q.float().permute(1, 0, 2)  # [Hq, Lq, D]
    kf = k.float().repeat_interleave(G, dim=0)
    vf = v.float().repeat_interleave(G, dim=0)
    s = torch.einsum("hqd,hkd->hqk", qf, kf) * scale
    kpos = torch.arange(Lk, device=q.device)[None, :]
    mask = kpos <= q_pos[:, None]
    if window and window > 0:
        mask = mask & (kpos > q_pos[:, None] - window)
    s = s.masked_fill(~mask[None], float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float()[:, None, None].expand(Hq, Lq, 1)], dim=-1)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    if sinks is not None:
        p = p[..., :-1]
    o = torch.einsum("hqk,hkd->hqd", p, vf)
    return o.permute(1, 0, 2).to(q.dtype)


def attn_decode(q, k_cache, v_cache, block_tables, ctx_lens, scale, window=0, sinks=None,
                max_ctx=0, num_splits=0, out=None, kv_scale=(1.0, 1.0)):
    B = q.shape[0]
    res = torch.zeros_like(q) if out is None else out
    for b in range(B):
        n = int(ctx_lens[b])
        if n <= 0:
            res[b] = 0
            continue
        k = _gather_kv(k_cache, block_tables[b], n, kv_scale[0])
        v = _gather_kv(v_cache, block_tables[b], n, kv_scale[1])
        pos = torch.tensor([n - 1], device=q.device)
        res[b] = _attend(q[b:b + 1], k, v, scale, pos, window, sinks)[0]
    return res


def attn_prefill(q, k_cache, v_cache, block_tables, cu_q, ctx_lens, max_q_len, scale, window=0,
                 sinks=None, out=None, kv_scale=(1.0, 1.0)):
    T, Hq, D = q.shape
    res = torch.zeros((T, Hq, D), dtype=q.dtype, device=q.device) if out is None else out
    B = ctx_lens.numel()
    for b in range(B):
        s, e = int(cu_q[b]), int(cu_q[b + 1])
        if e <= s:
            continue
        n = int(ctx_lens[b])
        prefix = n - (e - s)
        k = _gather_kv(k_cache, block_tables[b], n, kv_scale[0])
        v = _gather_kv(v_cache, block_tables[b], n, kv_scale[1])
        pos = prefix + torch.arange(e - s, device=q.device)
        res[s:e] = _attend(q[s:e], k, v, scale, pos, window, sinks)
    return res


def argmax(logits, want_logprob: bool = False):
    lf = logits.float()
    ids = lf.argmax(dim=-1).to(torch.int32)
    if want_logprob:
        lp = torch.log_softmax(lf, dim=-1).gather(1, ids.long()[:, None])[:, 0]
        return ids, lp
    return ids


def apply_penalties(logits, row_off, tok_ids, out_cnt, rep, pres, freq):
    """In place: repetition penalty on every listed token of a row (``l > 0 ? l / rep : l * rep``), frequency and
    presence penalties on the tokens that were generated (``l -= freq * count + pres``). Same rules as the GPU
    backends the reference forwards these parameters to (``src/parallax/sglang/batch_info.py:43-59``)."""
    B = logits.shape[0]
    for b in range(B):
        lo, hi = int(row_off[b]), int(row_off[b + 1])
        if hi <= lo:
            continue
        t = tok_ids[lo:hi].long()
        c = out_cnt[lo:hi].float()
        l = logits[b, t].float()
        r = float(rep[b])
        if r != 1.0:
            l = torch.where(l > 0, l / r, l * r)
        l = l - (c > 0).float() * (float(freq[b]) * c + float(pres[b]))
        logits[b, t] = l.to(logits.dtype)
    return logits


def patch_ids(dst, dst_idx, src, src_idx) -> None:
    """``dst[dst_idx] = src[src_idx]`` (in place)."""
    if dst_idx.numel():
        dst[dst_idx.long()] = src[src_idx.long()]


def sample(logits, temperature, top_k, top_p, min_p, uniform, want_prob: bool = False):
    """Sort-based sampler with the reference's filter order; one uniform number per row."""
    B, V = logits.shape
    lf = logits.float()
    ids = torch.empty(B, dtype=torch.int32, device=logits.device)
    probs_out = torch.empty(B, dtype=torch.float32, device=logits.device)
    for b in range(B):
        t = float(temperature[b])
        k = int(top_k[b])
        if t <= 0 or k == 1:
            i = int(lf[b].argmax())
            ids[b] = i
            probs_out[b] = torch.softmax(lf[b] / (t if t > 0 else 1.0), -1)[i]
            continue
        p = torch.softmax(lf[b] / t, dim=-1)
        ps, idx = torch.sort(p, descending=True, stable=True)
        csum = torch.cumsum(ps, 0)
        keep = torch.ones(V, dtype=torch.bool, device=logits.device)
        if k > 0:
            keep &= torch.arange(V, device=logits.device) < k
        keep &= (csum - ps) <= float(top_p[b])
        keep &= ps >= ps[0] * float(min_p[b])
        kept_ids = idx[keep]
        # draw in index order so that the same uniform number picks the same token as the kernel
        order = torch.sort(kept_ids).values
        w = p[order]
        c = torch.cumsum(w, 0)
        target = float(uniform[b]) * float(c[-1])
        j = int(torch.searchsorted(c, torch.tensor(target, device=c.device), right=True))
        j = min(j, order.numel() - 1)
        ids[b] = order[j].to(torch.int32)
        probs_out[b] = p[order[j]]
    return (ids, probs_out) if want_prob else ids


def moe_route(logits, e_bias, k, mode=0, renorm=True, n_group=1, topk_group=1, routed_scale=1.0):
    """Top-k expert selection (see csrc/moe.cu for the two modes)."""
    lf = logits.float()
    T, E = lf.shape
    if mode == 0:
        s = torch.softmax(lf, dim=-1)
        sel = s
    else:
        s = torch.sigmoid(lf)
        sel = s + (e_bias.float() if e_bias is not None else 0.0)
        if n_group > 1 and topk_group < n_group:
            g = sel.view(T, n_group, E // n_group)
            gscore = g.topk(2, dim=-1).values.sum(-1)
            keep = torch.zeros_like(gscore, dtype=torch.bool)
            keep.scatter_(1, gscore.topk(topk_group, dim=-1).indices, True)
            sel = g.masked_fill(~keep[:, :, None], float("-inf")).reshape(T, E)
    ids = sel.topk(k, dim=-1).indices
    w = s.gather(1, ids)
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return ids.to(torch.int32), (w * routed_scale).float()


def moe_ffn(x, ids, weights, w1, w2, num_experts, base=None, act_mode: int = 0, limit: float = 0.0, b1=None, b2=None):
    """Dense restatement: loop over experts. w1 ``[E*2I, H]`` (gate/up interleaved for act_mode 0,
    ``[gate | up]`` per expert otherwise), w2 ``[E*H, I]``, optional expert biases b1 / b2."""
    T, H = x.shape
    two_i = w1.shape[0] // num_experts
    w1e = w1.view(num_experts, two_i, H)
    w2e = w2.view(num_experts, H, two_i // 2)
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    for e in range(num_experts):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        if act_mode == 0:
            a = linear(x[tok], w1e[e], epi=EPI_SILU_MUL)
        else:
            gu = linear(x[tok], w1e[e], bias=None if b1 is None else b1.view(num_experts, two_i)[e])
            a = act_mul(gu, mode=act_mode, limit=limit)
        y = linear(a, w2e[e], bias=None if b2 is None else b2.view(num_experts, H)[e])
        out.index_add_(0, tok, y.float() * weights[tok, slot][:, None])
    if base is not None:
        out = out + base.float()
    return out.to(x.dtype)


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)


# ---------------------------------------------------------------------------- MLA / DSA
def _rope_interleaved(x, cos_sin, positions):
    """Rotate pairs (2i, 2i+1) of the last dim by the angle of ``positions`` (fp32)."""
    R = x.shape[-1]
    cs = cos_sin[positions.long()].float()                  # [T, R]
    cos, sin = cs[:, : R // 2], cs[:, R // 2:]
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    x0, x1 = x[..., 0::2].float(), x[..., 1::2].float()
    out = torch.stack([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)
    return out.flatten(-2)


def mla_kv_prep(ckv, norm_w, cos_sin, positions, slot_mapping, cache, eps, latent: int):
    """cache[slot] = [rmsnorm(ckv[:, :latent]) * w | rope_interleaved(ckv[:, latent:])]."""
    lat = ckv[:, :latent].float()
    lat = lat * torch.rsqrt(lat.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
    pe = _rope_interleaved(ckv[:, latent:], cos_sin, positions)
    rows = torch.cat([lat, pe], dim=-1).to(cache.dtype)
    flat = cache.view(-1, cache.shape[-1])
    ok = slot_mapping >= 0
    flat[slot_mapping[ok].long()] = rows[ok]


def mla_q_absorb(q, w_uk_s, cos_sin, positions, H: int, nope: int, latent: int):
    """q [T, H*(nope+R)] -> (q_lat_hm [H, Tpad, latent], q_pe [T, H, R]); w_uk_s [H*latent, nope]."""
    T = q.shape[0]
    q = q.view(T, H, -1)
    q_nope, q_pe = q[..., :nope], q[..., nope:]
    q_pe = _rope_interleaved(q_pe, cos_sin, positions).to(q.dtype)
    w = w_uk_s.view(H, latent, nope).float()
    q_lat = torch.einsum("thd,hcd->htc", q_nope.float(), w).to(q.dtype)
    return q_lat.contiguous(), q_pe.contiguous()


def mla_attn(q_lat_hm, q_pe, cache, block_tables, cu_q, positions, scale, tok_begin: int, n_tok: int, topk=None,
             out=None):
    """Absorbed latent attention for tokens [tok_begin, tok_begin + n_tok) -> o_lat_hm [H, Tpad, latent].
    ``positions`` / ``topk`` / ``q_pe`` rows are indexed by the batch-wide token index."""
    H, Tpad, L = q_lat_hm.shape
    page = cache.shape[-2]
    flat = cache.view(-1, cache.shape[-1]).float()
    if out is None:
        out = torch.zeros_like(q_lat_hm)
    cu = None if cu_q is None else cu_q.tolist()
    for t in range(tok_begin, tok_begin + n_tok):
        seq = t - tok_begin if cu is None else max(i for i in range(len(cu) - 1) if cu[i] <= t)
        pos = int(positions[t])
        if topk is not None and int(topk[t, 0]) >= 0:
            keys = topk[t]
            keys = keys[(keys >= 0) & (keys <= pos)].long()
        else:
            keys = torch.arange(pos + 1)
        bt = block_tables[seq].long()
        rows = flat[bt[keys // page] * page + keys % page]            # [n, L+R]
        ql = torch.cat([q_lat_hm[:, t].float(), q_pe[t].float()], dim=-1)   # [H, L+R]
        p = torch.softmax(ql @ rows.t() * scale, dim=-1)
        out[:, t] = (p @ rows[:, :L]).to(out.dtype)
    return out


def mla_unabsorb(o_lat_hm, w_uv_s, T: int):
    """o_lat_hm [H, Tpad, latent], w_uv_s [H*V, latent] -> [T, H*V]."""
    H, _Tpad, L = o_lat_hm.shape
    w = w_uv_s.view(H, -1, L).float()
    o = torch.einsum("htc,hvc->thv", o_lat_hm[:, :T].float(), w)
    return o.reshape(T, -1).to(o_lat_hm.dtype)


def store_rows(src, slot_mapping, cache):
    flat = cache.view(-1, cache.shape[-1])
    ok = slot_mapping >= 0
    flat[slot_mapping[ok].long()] = src[ok].to(cache.dtype)


def dsa_index_prep(q_idx, kv, k_off: int, w_off: int, ln_w, ln_b, ln_eps: float, cos_sin, positions, slot_mapping,
                   cache, w_scale: float, rope_dim: int):
    """Lightning-indexer pre-processing (``src/parallax/models/deepseek_v32.py:84-238``): interleaved rotation
    of the first ``rope_dim`` dims of every index-query head (in place on ``q_idx [T, Hi, Di]``), layer norm +
    rotation of the index key ``kv[:, k_off:k_off+Di]`` stored at ``cache[slot]``, head weights
    ``kv[:, w_off:w_off+Hi] * w_scale`` returned as fp32."""
    T, Hi, Di = q_idx.shape
    R = rope_dim
    q_idx[..., :R] = _rope_interleaved(q_idx[..., :R], cos_sin, positions).to(q_idx.dtype)
    ik = torch.nn.functional.layer_norm(kv[:, k_off:k_off + Di].float(), (Di,), ln_w.float(),
                                        None if ln_b is None else ln_b.float(), ln_eps)
    ik = torch.cat([_rope_interleaved(ik[:, :R], cos_sin, positions), ik[:, R:]], dim=-1).to(q_idx.dtype)
    store_rows(ik, slot_mapping, cache)
    return (kv[:, w_off:w_off + Hi].float() * w_scale).contiguous()


def dsa_index_scores(q_idx, w, index_cache, block_tables, cu_q, positions, max_ctx: int):
    """scores[t, j] = sum_h relu(q[t,h] . k_j) * w[t,h] for j <= positions[t], -inf beyond."""
    T = q_idx.shape[0]
    page = index_cache.shape[-2]
    flat = index_cache.view(-1, index_cache.shape[-1]).float()
    ld = (max_ctx + 63) // 64 * 64
    out = torch.full((T, ld), float("-inf"), dtype=torch.float32)
    cu = None if cu_q is None else cu_q.tolist()
    for t in range(T):
        seq = t if cu is None else max(i for i in range(len(cu) - 1) if cu[i] <= t)
        pos = int(positions[t])
        keys = torch.arange(pos + 1)
        bt = block_tables[seq].long()
        k = flat[bt[keys // page] * page + keys % page]               # [n, Di]
        s = torch.relu(q_idx[t].float() @ k.t())                        # [Hi, n]
        out[t, : pos + 1] = (s * w[t].float()[:, None]).sum(0)
    return out


def topk_select(scores, positions, k: int):
    """Positions of the k largest scores among [0, positions[t]]; rows with <= k candidates are -1."""
    T = scores.shape[0]
    out = torch.full((T, k), -1, dtype=torch.int32)
    for t in range(T):
        n = int(positions[t]) + 1
        if n > k:
            out[t] = torch.topk(scores[t, :n], k).indices.to(torch.int32)
    return out


# ---------------------------------------------------------------------------- block-scaled fp8
def quant_fp8_rows(x):
    from parallax_b200.loader.quant import quantize_fp8_rows

    return quantize_fp8_rows(x, 128)


def _dequant_w64(wq, w_s64):
    N, K = wq.shape
    s = w_s64.float().repeat_interleave(64, dim=0)[:N].repeat_interleave(128, dim=1)[:, :K]
    return wq.float() * s


def linear_fp8(x, wq, w_s64, residual=None, epi: int = EPI_NONE):
    """Same contraction as the fp8 kernel: activations are rounded to e4m3 per 1x128 group."""
    xq, xs = quant_fp8_rows(x)
    xd = xq.float() * xs.repeat_interleave(128, dim=1)[:, : x.shape[1]]
    y = xd @ _dequant_w64(wq, w_s64).t()
    if epi == EPI_SILU_MUL:
        N = wq.shape[0]
        yg = y.view(-1, N // 128, 2, 64)
        y = (torch.nn.functional.silu(yg[:, :, 0]) * yg[:, :, 1]).reshape(-1, N // 2)
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def moe_ffn_fp8(x, ids, weights, w1q, w1s, w2q, w2s, num_experts: int, base=None):
    T, H = x.shape
    n1, n2 = w1q.shape[0] // num_experts, w2q.shape[0] // num_experts
    out = torch.zeros(T, n2, dtype=torch.float32) if base is None else base.float().clone()
    for e in range(num_experts):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        a = linear_fp8(x[tok], w1q[e * n1:(e + 1) * n1], w1s[e * n1 // 64:(e + 1) * n1 // 64], epi=EPI_SILU_MUL)
        y = linear_fp8(a, w2q[e * n2:(e + 1) * n2], w2s[e * n2 // 64:(e + 1) * n2 // 64])
        out.index_add_(0, tok, y.float() * weights[tok, slot].float()[:, None])
    return out.to(x.dtype)


# ---------------------------------------------------------------------------- gated delta net
def causal_conv1d_silu(x, w, bias, conv_state, seq_cu, seq_slots, positions):
    """Per-channel causal convolution + SiLU with the last K-1 inputs carried per request slot."""
    T, C = x.shape
    K = w.shape[1]
    out = torch.empty((T, C), dtype=x.dtype)
    cu = seq_cu.tolist()
    wf = w.float()
    for b in range(len(cu) - 1):
        t0, t1 = cu[b], cu[b + 1]
        if t1 <= t0:
            continue
        slot = int(seq_slots[b])
        hist = torch.zeros(K - 1, C) if int(positions[t0]) == 0 else conv_state[slot].float().t()
        u = torch.cat([hist, x[t0:t1].float()], dim=0)                 # [K-1+n, C]
        win = u.unfold(0, K, 1)                                        # [n, C, K]
        y = (win * wf[None]).sum(-1)
        if bias is not None:
            y = y + bias.float()
        out[t0:t1] = torch.nn.functional.silu(y).to(x.dtype)
        conv_state[slot] = u[-(K - 1):].t().to(conv_state.dtype)
    return out


def gated_delta_rule(qkv, a, b, A_log, dt_bias, z, norm_w, rec_state, seq_cu, seq_slots, positions, Hk: int, Hv: int,
                     Dk: int, Dv: int, eps: float):
    """Sequential gated delta rule with a per-request state ``[Hv, Dv, Dk]`` and gated RMSNorm."""
    T = qkv.shape[0]
    out = torch.empty((T, Hv * Dv), dtype=qkv.dtype)
    cu = seq_cu.tolist()
    rep = Hv // Hk
    for s in range(len(cu) - 1):
        t0, t1 = cu[s], cu[s + 1]
        if t1 <= t0:
            continue
        slot = int(seq_slots[s])
        S = torch.zeros(Hv, Dv, Dk) if int(positions[t0]) == 0 else rec_state[slot].float().clone()
        for t in range(t0, t1):
            row = qkv[t].float()
            q = row[:Hk * Dk].view(Hk, Dk)
            k = row[Hk * Dk:2 * Hk * Dk].view(Hk, Dk)
            v = row[2 * Hk * Dk:].view(Hv, Dv)
            q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) / Dk ** 0.5
            k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
            q, k = q.repeat_interleave(rep, 0), k.repeat_interleave(rep, 0)        # [Hv, Dk]
            g = -torch.exp(A_log.float()) * torch.nn.functional.softplus(a[t].float() + dt_bias.float())
            beta = torch.sigmoid(b[t].float())
            S = S * torch.exp(g)[:, None, None]
            mem = torch.einsum("hvk,hk->hv", S, k)
            d = (v - mem) * beta[:, None]
            S = S + d[:, :, None] * k[:, None, :]
            o = torch.einsum("hvk,hk->hv", S, q)
            zz = z[t].float().view(Hv, Dv)
            y = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float() * torch.nn.functional.silu(zz)
            out[t] = y.reshape(-1).to(out.dtype)
        rec_state[slot] = S.to(rec_state.dtype)
    return out


def sigmoid_gate_mul(x, gate):
    return (x.float() * torch.sigmoid(gate.float())).to(x.dtype)


def gate_mul_grouped(x, gate, group: int, residual=None):
    T, N = x.shape
    y = (x.float().view(T, N // group, group) * torch.sigmoid(gate.float()).view(T, N // group, 1)).view(T, N)
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def row_dot(x, w):
    return (x.float() @ w.float().view(-1, 1)).to(x.dtype)


# ---------------------------------------------------------------------------- block-sparse indexer (MSA)
def msa_block_scores(iq, index_cache, block_tables, cu_q, positions, max_ctx: int, sparse_block: int, scale: float):
    """scores[t, j] = max over index heads and visible tokens of block j of scale * iq . ik."""
    T = iq.shape[0]
    page = index_cache.shape[-2]
    flat = index_cache.view(-1, index_cache.shape[-1]).float()
    nb = (max_ctx + sparse_block - 1) // sparse_block
    out = torch.full((T, nb), float("-inf"), dtype=torch.float32)
    cu = None if cu_q is None else cu_q.tolist()
    for t in range(T):
        seq = t if cu is None else max(i for i in range(len(cu) - 1) if cu[i] <= t)
        pos = int(positions[t])
        keys = torch.arange(pos + 1)
        bt = block_tables[seq].long()
        k = flat[bt[keys // page] * page + keys % page]
        s = (iq[t].float() @ k.t() * scale).max(0).values                 # [pos+1]
        for j in range(pos // sparse_block + 1):
            out[t, j] = s[j * sparse_block:(j + 1) * sparse_block].max()
    return out


def msa_select(scores, positions, block_tables, cu_q, page: int, sparse_block: int, topk: int, init_blocks: int,
               local_blocks: int):
    """Top-k causal blocks per query (forced init/local blocks) -> virtual block table + visible tokens."""
    T = scores.shape[0]
    ppb = sparse_block // page
    v_tables = torch.zeros((T, topk * ppb), dtype=torch.int32)
    v_ctx = torch.empty(T, dtype=torch.int32)
    cu = None if cu_q is None else cu_q.tolist()
    for t in range(T):
        seq = t if cu is None else max(i for i in range(len(cu) - 1) if cu[i] <= t)
        pos = int(positions[t])
        cur = pos // sparse_block
        s = scores[t, :cur + 1].clone()
        s[torch.isnan(s)] = float("-inf")
        s[:init_blocks] = 1e30
        s[max(cur - local_blocks + 1, 0):] = 1e29
        k = min(topk, cur + 1)
        # arg-max rounds with ties to the lower index (stable sort by descending score)
        order = torch.sort(s, descending=True, stable=True).indices[:k]
        blocks = torch.sort(order).values
        pages = (blocks[:, None] * ppb + torch.arange(ppb)[None]).reshape(-1)
        bt = block_tables[seq].long()
        v_tables[t, : k * ppb] = torch.where(pages < bt.shape[0], bt[pages.clamp_max(bt.shape[0] - 1)],
                                             torch.zeros_like(pages)).int()
        v_ctx[t] = (k - 1) * sparse_block + pos - cur * sparse_block + 1
    return v_tables, v_ctx
