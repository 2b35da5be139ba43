"""The allocation-free RMSNorm backward (``mb_rmsnorm_bwd_static``) against the regular entry point.

The exported C symbol is called through ctypes exactly as a C host would call it; the scratch the regular entry point
receives from the caller lives in a static device array inside the library instead. Collected last (file name) so it
also runs after every other GPU test has used the library in the same process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_H, MAX_BLOCKS = 8192, 304


def _run_both(rows, H, with_residual, seed):
    from maltos_b200.ops import _lib

    L = _lib.lib()
    fn = L.mb_rmsnorm_bwd_static
    fn.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(seed)
    dy = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    h = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=dev, generator=g)).bfloat16()
    dres = torch.randn(rows, H, device=dev, generator=g).bfloat16() if with_residual else None
    rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-5).contiguous()

    nblk = L.mb_rmsnorm_bwd_blocks(_lib.c_ll(rows))
    partial = torch.empty((nblk, H), device=dev, dtype=torch.float32)
    dx_ref, dw_ref = torch.empty_like(h), torch.empty_like(w)
    dwf_ref = torch.zeros(H, device=dev, dtype=torch.float32)
    _lib.check(L.mb_rmsnorm_bwd(_lib.ptr(dy), _lib.ptr(h), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres), _lib.ptr(dx_ref),
                                _lib.ptr(partial), _lib.ptr(dw_ref), _lib.ptr(dwf_ref), _lib.c_int(0), _lib.c_ll(rows),
                                _lib.c_int(H), _lib.stream_ptr()), "mb_rmsnorm_bwd")

    dx, dw = torch.full_like(h, float("nan")), torch.full_like(w, float("nan"))
    dwf = torch.full((H,), float("nan"), device=dev, dtype=torch.float32)
    before = torch.cuda.memory_allocated(dev)
    rc = fn(_lib.ptr(dy), _lib.ptr(h), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(dw),
            _lib.ptr(dwf), _lib.c_int(0), _lib.c_ll(rows), _lib.c_int(H), _lib.stream_ptr())
    _lib.check(rc, "mb_rmsnorm_bwd_static")
    torch.cuda.synchronize(dev)
    assert torch.cuda.memory_allocated(dev) == before

    # plain fp32 formulation of the same op
    hf, wf, dyf = h.float(), w.float(), dy.float()
    xhat = hf * rstd[:, None]
    gy = dyf * wf
    dx_f = rstd[:, None] * (gy - xhat * (gy * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx_f = dx_f + dres.float()
    dw_f = (dyf * xhat).sum(0)
    return (dx, dw, dwf), (dx_ref, dw_ref, dwf_ref), (dx_f, dw_f)


@pytest.mark.parametrize("rows,H,with_residual", [(1000, 4096, True), (37, 512, False), (4096, 8192, False)])
def test_static_scratch_matches_regular_entry_point(rows, H, with_residual):
    for call in range(2):   # two calls in a row reuse the same scratch
        got, ref, fp32 = _run_both(rows, H, with_residual, seed=call)
        for a, b in zip(got, ref):
            assert torch.isfinite(a.float()).all()
            torch.testing.assert_close(a.float(), b.float(), rtol=0, atol=0)   # same kernels, same block order
        dx_f, dw_f = fp32
        assert (got[0].float() - dx_f).abs().max() <= 2e-2 * dx_f.abs().max()
        assert (got[1].float() - dw_f).abs().max() <= 2e-2 * dw_f.abs().max()
        assert (got[2] - dw_f).abs().max() <= 1e-3 * dw_f.abs().max()
    from maltos_b200.ops import _lib

    _lib.fetch_status()


def test_rejects_problem_beyond_static_scratch():
    from maltos_b200.ops import _lib

    L = _lib.lib()
    fn = L.mb_rmsnorm_bwd_static
    fn.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    H = MAX_H + 8
    t = torch.zeros(4, H, device=dev, dtype=torch.bfloat16)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    rstd = torch.ones(4, device=dev)
    dx = torch.zeros_like(t)
    dw = torch.zeros_like(w)
    rc = fn(_lib.ptr(t), _lib.ptr(t), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(None), _lib.ptr(dx), _lib.ptr(dw),
            _lib.c_void_p(0), _lib.c_int(0), _lib.c_ll(4), _lib.c_int(H), _lib.stream_ptr())
    assert rc == -2
    assert b"static scratch" in L.mb_last_error()
    rc = fn(_lib.ptr(t), _lib.ptr(t), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(None), _lib.ptr(dx), _lib.ptr(dw),
            _lib.c_void_p(0), _lib.c_int(0), _lib.c_ll(4), _lib.c_int(12), _lib.stream_ptr())
    assert rc == -1
    assert float(dx.abs().sum()) == 0.0   # nothing was launched
