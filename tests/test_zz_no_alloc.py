"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory when they call it (they run
inside a pool someone else owns, or their serving loop bans allocator calls after start-up).
``pxl_attn_decode_static_scratch`` serves them with a scratch array built into the library.
This test checks it against the regular entry point, which gets its scratch from the caller,
on two calls in a row (the second call reuses the array with the first call's leftovers in it).

The file name keeps it last in collection order, so a run that stops at the first failure has
already run every other test.
"""

import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind():
    from parallax_b200.ops import _lib

    fn = _lib.lib().pxl_attn_decode_static_scratch
    fn.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_float, c_int, c_int,
                   c_void_p, c_void_p]
    fn.restype = c_int
    return fn


def _case(seed, B, ctx_max, Hq=32, Hkv=8, D=128, page=16):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(seed)
    ctx = torch.randint(1, ctx_max + 1, (B,), generator=g).tolist()
    nb = [(n + page - 1) // page for n in ctx]
    total = sum(nb) + 2
    perm = torch.randperm(total, generator=g).to(torch.int32)
    bt = torch.zeros(B, max(nb), dtype=torch.int32)
    o = 0
    for b, n in enumerate(nb):
        bt[b, :n] = perm[o:o + n]
        o += n
    torch.manual_seed(seed)
    kc = torch.randn(total, Hkv, page, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(total, Hkv, page, D, device=dev, dtype=torch.bfloat16)
    q = torch.randn(B, Hq, D, device=dev, dtype=torch.bfloat16)
    return q, kc, vc, bt.to(dev), torch.tensor(ctx, dtype=torch.int32, device=dev)


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def test_static_scratch_matches_regular_entry_point_twice():
    from parallax_b200.ops import cuda as cu

    fn = _bind()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = cu.status_tensor(dev)
    for call, (seed, B, ctx_max, splits) in enumerate([(11, 6, 900, 4), (12, 9, 400, 3)]):
        q, kc, vc, bt, cl = _case(seed, B, ctx_max)
        Hq, D = q.shape[1], q.shape[2]
        scale = 1.0 / math.sqrt(D)
        want = cu.attn_decode(q, kc, vc, bt, cl, scale, num_splits=splits, max_ctx=ctx_max)
        got = torch.full_like(q, float("nan"))
        rc = fn(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), cl.data_ptr(),
                got.data_ptr(), None, B, Hq, kc.shape[1], D, kc.shape[2], bt.shape[1], kc.shape[0],
                scale, 0, splits, status.data_ptr(), stream)
        assert rc == 0, f"call {call}: rc={rc}"
        torch.cuda.synchronize()
        cu.check_status(dev)
        assert torch.isfinite(got.float()).all()
        assert _rel_err(got, want) < 2e-2, f"call {call}"
        # same kernels, same split count: the two paths should agree far tighter than that
        assert torch.allclose(got.float(), want.float(), atol=1e-2, rtol=1e-2)


def test_static_scratch_head_dim_64_takes_the_cp_async_kernel():
    """Head dim 64 (and page size 8) is outside the TMA-fed kernel: the same entry point then runs the
    cp.async kernel over the same built-in scratch, against the fp32 restatement."""
    from parallax_b200.ops import cuda as cu
    from parallax_b200.ops import reference as ref

    fn = _bind()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = cu.status_tensor(dev)
    q, kc, vc, bt, cl = _case(21, 7, 500, Hq=16, Hkv=4, D=64, page=8)
    scale = 1.0 / math.sqrt(64)
    want = ref.attn_decode(q, kc, vc, bt, cl, scale)
    for splits in (1, 3):
        got = torch.full_like(q, float("nan"))
        rc = fn(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), cl.data_ptr(),
                got.data_ptr(), None, q.shape[0], 16, 4, 64, 8, bt.shape[1], kc.shape[0], scale, 0, splits,
                status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        cu.check_status(dev)
        assert _rel_err(got, want) < 2e-2, splits


def test_static_scratch_rejects_oversize_and_bad_splits():
    fn = _bind()
    q, kc, vc, bt, cl = _case(13, 4, 64)
    args = lambda B, splits: (q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(),
                              cl.data_ptr(), q.data_ptr(), None, B, 32, 8, 128, 16, bt.shape[1],
                              kc.shape[0], 0.1, 0, splits, None, None)
    # 4096 sequences x 32 heads x 64 splits x 130 floats is far beyond the 4 Mi-float array:
    # refused up front, nothing is launched (the pointers are never dereferenced)
    assert fn(*args(4096, 64)) == 4
    assert fn(*args(4, 0)) == 1
